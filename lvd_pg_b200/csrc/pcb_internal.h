// pcb_internal.h — data layout of a compiled circuit in HBM, shared by the translation units
// of libpcb200.so.
//
// Layout decisions (all ids 0-based on the device):
//  * Work matrices (mars, flows, klds, ...) are node-major with the example index contiguous:
//    element (b, n) at n*ld + b, ld a multiple of 32 floats.  This is the reference's column-major
//    [B, N] matrix with a padded leading dimension, so a warp that covers 32 examples of one node
//    reads and writes 128 contiguous bytes.
//  * Parameters live in ONE flat vector `theta` in the reference's flat order
//    (sum-edge log-params in up-edge order, then the log-probs of learnable leaves in input-node
//    order; log-probs of fixed leaves are appended behind it).  vectorize/update_parameters are
//    plain copies and KLD / Adam / sampling read the same vector the EM step updates.
//  * Sufficient statistics live in ONE flat vector `aggr` = [edge flows by param id |
//    leaf flow slots (C+1 per learnable leaf) | batch log-likelihood sum], which is exactly the
//    buffer the multi-GPU step all-reduces.
//  * A dense block is a run of R sum nodes with consecutive ids that all have the same K children
//    (prime ids c0..c0+K-1, optional sub ids d0..d0+K-1); its R*K parameters are consecutive in
//    theta (row = parent, child index fastest).  HCLT latent transitions are such blocks.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>
#include <string>
#include <mutex>
#include <vector>

#include "../../include/pcb200.h"

#define PCB_NONE 0xffffffffu
#define PCB_LEAF_CHUNK 8
#define PCB_LEAF_GROUP 64

struct PcbDenseBlock {
  uint32_t p0;    // first parent node
  uint32_t R;     // number of parents
  uint32_t K;     // number of children
  uint32_t c0;    // first prime child
  uint32_t d0;    // first sub child or PCB_NONE
  uint32_t pid0;  // first parameter id
  uint32_t mx_row;  // row of the per-block max buffer in the workspace
  uint32_t pad;
};

// Where a dense block's weight images live (floats into w_img): exp(theta) split into TF32 hi/lo
// and stored as operand tiles [column tile][K chunk][hi | lo][rows x 32 floats, 128-byte swizzle].
// off_f / rows_f / nch_f: rows = parents, K = children (forward); off_t / ...: the transpose.
struct PcbDenseImg {
  uint64_t off_f, off_t;
  uint32_t rows_f, rows_t, nch_f, nch_t;
};

// incoming-edge entry of a node (CSR by child, used by every top-down pass)
struct PcbInEntry {
  uint32_t parent;
  uint32_t sib;   // the other child of the edge or PCB_NONE
  uint32_t pid;   // parameter id of a sum edge, PCB_NONE for product edges
  uint32_t flags; // bit0: this node is the prime child of the edge (aggregating entry)
};

// kernel classes for launch counting and the optional per-class event timing
enum PcbKernelClass {
  PCB_K_LEAF_FWD = 0, PCB_K_SPARSE_UP, PCB_K_DENSE_FWD, PCB_K_SPARSE_DOWN, PCB_K_DENSE_BWD_CHILD,
  PCB_K_DENSE_BWD_EDGE, PCB_K_LEAF_FLOW, PCB_K_UPDATE, PCB_K_MISC, PCB_K_ALLREDUCE, PCB_K_DENSE_MAX,
  PCB_K_W_IMAGE, PCB_K_KLD, PCB_K_SAMPLE, PCB_K_COUNT
};
struct PcbProfEvent { int cls; cudaEvent_t e0, e1; };
struct PcbProf {
  bool on = false;
  uint64_t launches[PCB_K_COUNT] = {0};
  std::vector<PcbProfEvent> ev;
};

struct pcb_circuit {
  int device = 0;
  PcbProf prof;
  uint32_t N = 0, E = 0, V = 0, L = 0;  // nodes, edges, variables, up layers (layer 0 = inputs)
  uint32_t n_inner = 0, n_input_params = 0, n_groups = 0, n_inputs = 0;
  uint32_t n_regions = 0, max_group = 0, max_cats = 0;
  uint64_t P = 0;            // n_inner + n_input_params
  uint64_t theta_len = 0;    // P + log-probs of fixed leaves
  uint64_t n_leaf_flow = 0;  // total leaf flow slots
  uint64_t aggr_len = 0;     // n_inner + n_leaf_flow + 1
  uint64_t dense_edges = 0;
  uint64_t device_bytes = 0;

  // ---- device arrays ----
  float* theta = nullptr;
  float* aggr = nullptr;
  uint8_t* kind = nullptr;        // [N]
  uint32_t* n_estart = nullptr;   // [N] first up-edge of an inner node
  uint32_t* n_ecount = nullptr;   // [N]
  uint32_t* n_pid0 = nullptr;     // [N] first parameter id of a sum node
  uint32_t* n_region = nullptr;   // [N] 0-based sum region or PCB_NONE
  uint32_t* e_prime = nullptr;    // [E]
  uint32_t* e_sub = nullptr;      // [E]
  // leaves, indexed by input index i (input_node_ids order)
  uint32_t* in_node = nullptr;    // [n_inputs] node id
  uint32_t* in_var = nullptr;     // [n_inputs] 0-based variable
  uint32_t* in_cats = nullptr;    // [n_inputs]
  uint64_t* in_poff = nullptr;    // [n_inputs] offset of the log-probs in theta
  uint64_t* in_foff = nullptr;    // [n_inputs] offset of the flow slots in aggr, ~0 for fixed
  uint32_t* node2input = nullptr; // [N] input index or PCB_NONE
  // multi-head circuits: heads = children of the fake root's skipped edges, in edge order
  uint32_t* n_head = nullptr;     // [N] head index or PCB_NONE
  uint32_t* head_roots = nullptr; // [n_heads] node ids
  std::vector<uint32_t> h_head_roots;
  uint32_t n_heads = 0;
  // live workspaces of this circuit: their captured step graphs hold references to the communicator
  std::vector<pcb_workspace*> workspaces;
  std::mutex ws_mu;
  // packed per-node and per-leaf records for the sampling walk (one 16-byte load per visited node):
  // node: {first edge, edge count, first parameter id (sum) or input index (leaf), kind | region << 2}
  // leaf: {parameter offset lo, hi, categories, variable}
  uint4* s_node = nullptr;        // [N]
  uint4* s_leaf = nullptr;        // [n_inputs]
  // leaves grouped by variable and cut into chunks of at most PCB_LEAF_CHUNK: one thread block
  // stages the variable's observed values once and serves every leaf of the chunk
  uint32_t* lchunk_var = nullptr;   // [n_lchunks] variable of the chunk
  uint32_t* lchunk_off = nullptr;   // [n_lchunks + 1] range into lchunk_inputs
  uint32_t* lchunk_inputs = nullptr; // [n_inputs] input indices sorted by variable
  uint32_t n_lchunks = 0;
  // the same order cut into groups of at most PCB_LEAF_GROUP leaves of one variable (leaf statistics)
  uint32_t* lgrp_var = nullptr;
  uint32_t* lgrp_off = nullptr;
  uint32_t n_lgrps = 0;
  // layer lists: all inner nodes by layer / only those outside dense blocks
  uint32_t* up_all = nullptr;     // [n_inner_nodes]
  uint8_t* up_same = nullptr;     // per chunk of 8 entries of a layer of up_all: same children in the same order
  std::vector<uint32_t> h_up_chunk_off;   // [L+1] first chunk of a layer (index = layer-1)
  uint32_t* up_sparse = nullptr;
  uint32_t* down_all = nullptr;   // [N] every node, by layer
  uint32_t* down_sparse = nullptr;
  uint32_t* in_off = nullptr;     // [N+1] CSR by child
  PcbInEntry* in_ent = nullptr;
  PcbDenseBlock* dense = nullptr; // sorted by parent layer
  uint32_t* grp_node = nullptr;   // [n_groups] sum node of each parameter group

  // ---- host copies of the small per-layer tables ----
  std::vector<uint32_t> h_up_all_off, h_up_sparse_off;      // [L+1] (index = layer-1)
  std::vector<uint32_t> h_down_all_off, h_down_sparse_off;  // [L+2] (index = layer)
  std::vector<uint32_t> h_dense_off;                        // [L+1] blocks by parent layer
  std::vector<PcbDenseBlock> h_dense;
  uint32_t n_dense = 0;
  uint32_t max_dense_K = 0, max_dense_R = 0;

  // ---- host data kept for accessors ----
  std::vector<uint32_t> h_down2up;       // 0-based
  std::vector<uint32_t> h_edge2param;    // [E] 1-based pid or 0
  std::vector<uint32_t> h_region1;       // [N] 1-based region or 0
  std::vector<uint32_t> h_in_node, h_in_cats, h_heap_start;
  std::vector<uint8_t> h_in_fixed;
  std::vector<uint64_t> h_in_poff, h_in_foff;
  uint64_t heap_len = 0;

  // ---- dense-block implementation and the device status word bounded waits report to ----
  bool use_tc = false;
  float* w_img = nullptr;
  PcbDenseImg* dense_img = nullptr;
  uint64_t w_img_len = 0;
  bool w_img_valid = false;
  // 16-deep weight images of the kernels that read the data-dependent operand example-major
  // (pcb_dense_mn.cu); tc_mn selects those kernels for values and child flows
  bool tc_mn = true;
  float* w_img16 = nullptr;
  PcbDenseImg* dense_img16 = nullptr;
  uint64_t w_img16_len = 0;
  // edge statistics feed nothing downstream in the backward pass, so their kernels run on a
  // side stream, forked from and joined to the caller's stream with two reusable events
  cudaStream_t side = nullptr;
  cudaEvent_t ev_fork = nullptr, ev_join = nullptr;
  bool side_busy = false;
  // second side stream: the sparse nodes of layer l-1 take their flows while the dense blocks of layer l run
  cudaStream_t side2 = nullptr;
  cudaEvent_t ev_fork2 = nullptr, ev_join2 = nullptr;
  cudaStream_t gstream = nullptr;   // stands in for the legacy default stream, which cannot be captured
  cudaEvent_t ev_g0 = nullptr, ev_g1 = nullptr;
  bool graph_enabled = true;
  bool pdl = true;   // chain kernels are launched with programmatic stream serialization
  // tuning switches, read from the environment once when the circuit is created
  bool fwd_split = true, bwd_split = true;   // side-stream splits of the forward / backward layer loops
  bool early_update = false;                 // single-GPU step: sum update + weight images beside the leaf statistics (measured neutral)
  int leaf_flow_impl = 0;                    // 0 by category count, 1 shared-memory histograms, 2 sorted segments
  bool checked = false;                      // PCB_CHECKED=1: every pass first validates the batch (row ids, categories) and synchronises
  uint32_t* var_cats = nullptr;              // [V] smallest category count over a variable's leaves
  int32_t* check_word = nullptr;             // [4] first finding of the validation kernel: code, example, variable, value
  int tc_ksplit = 0;                         // 0 automatic, else 1 / 2 / 4 K parts of a dense tile (PCB_TC_KSPLIT)
  int tc_nsplit = 0;                         // 0 automatic, else 1 / 2 / 4 column splits of a dense tile
  int tc_a_stages = 0;                       // 0 automatic, else 2 / 4 / 8 stages of the dense kernels' A ring
  bool edge_ld = false;                      // edge statistics by the load-fed kernel instead of tensor-map copies
  bool sample_walk_warp = false;             // hard sampling: one warp per sample (the stack walk) instead of one CTA
  bool sample_exact_keys = false;            // hard sampling: every key in fp64 (cross-check of the fp32 pre-selection)
  // dense blocks [edge_lo, edge_hi) whose edge statistics are still to be launched, and the number
  // of tiles at which the range is launched
  uint32_t edge_lo = 0, edge_hi = 0, edge_batch_tiles = 592;
  int* status = nullptr;
  bool skip_stats = false;   // set around a backward pass that wants the flows only (no edge / leaf statistics)

  // ---- multi-GPU ----
  void* comm = nullptr;  // ncclComm_t
  int nranks = 1, rank = 0;
  bool comm_lost = false;                // pcb_comm_abort ran: steps refuse until the communicator is destroyed
  bool comm_enabled = true;             // false: the step skips its collectives (timing of the exposed share only)
  bool comm_pipe = true;                // sum parameters updated and weight images rebuilt while the leaf slots are summed (PCB_COMM_PIPE=0: one collective, then the update)
  bool comm_split = false;              // edge statistics summed on comm_stream while the leaf statistics are still formed
  cudaStream_t comm_stream = nullptr;   // created with the communicator
  cudaEvent_t ev_c0 = nullptr, ev_c1 = nullptr, ev_c2 = nullptr, ev_c3 = nullptr;
};

struct pcb_workspace {
  pcb_circuit* c = nullptr;
  uint32_t max_batch = 0, ld = 0;
  float* mars = nullptr;    // [N][ld]
  float* flows = nullptr;   // [N][ld]
  float* blk_mx = nullptr;  // [n_dense][ld] per-example max of a dense block's children
  float* mn_part = nullptr;        // partial tiles of the dense kernels' K split (296 slots of 128 x 257 floats)
  uint32_t* mn_tickets = nullptr;  // arrival counter per K-split tile, zero between launches
  // One EM step as a CUDA graph: a step called twice in a row with the same arguments is captured
  // on the second call and replayed from then on (the row ids are staged in ids_stage so that
  // their address does not change from step to step).
  struct StepKey {
    const void* data; const void* miss; const void* weights; void* comm; void* stream;
    const void* soft; const void* head_mask; float soft_reg; uint32_t soft_width; uint32_t comm_on;
    uint64_t num_rows;
    uint32_t row_start, B;
    float clear_rate, pseudocount, inertia;
    uint32_t has_ids, w_valid;
  };
  StepKey last_key{}, exec_key{};
  bool have_key = false;
  cudaGraphExec_t step_exec = nullptr;
  uint64_t step_launches[PCB_K_COUNT] = {0};   // launches of one replay, per kernel class
  int32_t* ids_stage = nullptr;                 // [max_batch]
  bool exec_end_w_valid = false;                // w_img_valid after a replay of step_exec
  float* ll_tmp = nullptr;                      // [max_batch] per-example log-likelihoods of a multi-head step
  // tensor maps over mars / flows for the copy-fed edge-statistics kernel (128-byte opaque objects)
  alignas(64) unsigned char tm[3][128];
  bool have_tm = false;
  // tensor map over mars with boxes of [16 rows][128 examples] (row slabs of the values / child-flow kernels)
  alignas(64) unsigned char tm_rows[128];
  bool have_tm_rows = false;
  // state of the last forward
  uint32_t B = 0;
  const uint8_t* data = nullptr;
  const uint8_t* miss = nullptr;
  uint64_t num_rows = 0;
  const int32_t* row_ids = nullptr;
  uint32_t row_start = 1;
  bool have_forward = false;
  const float* soft = nullptr;        // soft evidence [num_rows, V, C] or null
  const float* head_mask = nullptr;   // [num_rows, n_heads] or null
  float soft_reg = 0.0f;
  uint32_t soft_width = 1;
  // per-parameter-set buffers, allocated on first use
  uint32_t S_cap = 0, ldS = 0, stack_S = 0;
  int32_t* sample_status = nullptr;   // status word of the hard sampler's walk
  float* klds = nullptr;     // [N][ldS]
  float* grads = nullptr;    // [N][ldS]  (also td_probs)
  float* eprob = nullptr;    // [n_inner][ldS]
  float* cum = nullptr;      // [n_groups][ldS]
  uint32_t* stack = nullptr; // [S_cap][stack_cap]
  uint32_t stack_cap = 0;
  uint32_t kld_S = 0;
  bool have_kld = false;
  // the fused KLD + gradient + Adam step (pcb_kld_adam_step): gradient buffers, the device word that
  // holds the step count, and the captured chain
  int* kld_t_dev = nullptr;
  int* kld_bump = nullptr;   // set while the fused step runs: the leaf kernel counts the step here
  int32_t kld_t_host = -1;
  struct KldKey {
    const void* q; const void* p; const void* m; const void* v; const void* out; void* stream;
    float lr, b1, b2, eps;
  };
  KldKey kld_last_key{}, kld_exec_key{};
  bool have_kld_key = false;
  cudaGraphExec_t kld_exec = nullptr;
  uint64_t kld_launches[PCB_K_COUNT] = {0};
};

// ---- helpers ----
void pcb_set_error(const std::string& msg);
int32_t pcb_fail(int32_t code, const std::string& msg);

#define PCB_CUDA(expr)                                                                     \
  do {                                                                                     \
    cudaError_t _e = (expr);                                                               \
    if (_e != cudaSuccess)                                                                 \
      return pcb_fail(PCB_ERR_CUDA, std::string(#expr) + ": " + cudaGetErrorString(_e));   \
  } while (0)

#define PCB_REQUIRE(cond, msg) \
  do {                         \
    if (!(cond)) return pcb_fail(PCB_ERR_INVALID, msg); \
  } while (0)

static inline uint32_t pcb_round_up(uint32_t x, uint32_t m) { return (x + m - 1) / m * m; }

// cudaFuncSetAttribute applies to the current device only: a kernel that needs more than 48 KB of
// dynamic shared memory is configured once per device it is launched on (a host may hold circuits
// on several GPUs in one process).  Two threads racing here both set the same value.
struct PcbPerDeviceOnce {
  std::atomic<uint64_t> done{0};
  template <typename F>
  cudaError_t run(F&& configure) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    const uint64_t bit = 1ull << (dev & 63);
    if (done.load(std::memory_order_acquire) & bit) return cudaSuccess;
    e = configure();
    if (e == cudaSuccess) done.fetch_or(bit, std::memory_order_release);
    return e;
  }
};

// Counts a launch of class `cls`; with profiling on, brackets it with two events on `st`.
// A build with -DPCB_NVTX additionally wraps every launch scope (and the passes of a step, PcbNvtxRange) in an
// NVTX range named after its kernel class, for timeline tools; the default build has no NVTX calls.
#ifdef PCB_NVTX
#include <nvtx3/nvToolsExt.h>
struct PcbNvtxRange {
  explicit PcbNvtxRange(const char* name) { nvtxRangePushA(name); }
  ~PcbNvtxRange() { nvtxRangePop(); }
};
#else
struct PcbNvtxRange { explicit PcbNvtxRange(const char*) {} };
#endif
extern "C" const char* pcb_profile_class_name(int32_t i);

struct PcbProfScope {
  pcb_circuit* c; cudaStream_t st; cudaEvent_t e1 = nullptr;
  PcbNvtxRange nvtx;
  PcbProfScope(pcb_circuit* c_, cudaStream_t st_, int cls) : c(c_), st(st_), nvtx(pcb_profile_class_name(cls)) {
    ++c->prof.launches[cls];
    if (c->prof.on) {
      cudaEvent_t e0;
      cudaEventCreate(&e0); cudaEventCreate(&e1);
      cudaEventRecord(e0, st);
      c->prof.ev.push_back(PcbProfEvent{cls, e0, e1});
    }
  }
  ~PcbProfScope() { if (e1) cudaEventRecord(e1, st); }
};

// Launch with programmatic stream serialization: the kernel may be scheduled while its predecessor
// in the stream is still running, so its set-up (barrier initialisation, tensor-memory allocation)
// overlaps the predecessor's tail.  Such a kernel executes pcb_grid_dep_wait() before it touches
// global memory that an earlier kernel writes or reads, and pcb_grid_dep_launch() on entry.
template <typename... KArgs, typename... Args>
inline cudaError_t pcb_launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st,
                                  bool pdl, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr; cfg.numAttrs = pdl ? 1u : 0u;
  return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}
#ifdef __CUDACC__
__device__ __forceinline__ void pcb_grid_dep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pcb_grid_dep_launch() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
#endif

// entry points implemented across translation units and used by pcb_em_step
int32_t pcb_allreduce_aggr(pcb_circuit* c, cudaStream_t st);
// checked mode: validates row ids and categories of a batch, synchronises, PCB_ERR_INVALID with the first finding
int32_t pcb_check_batch(pcb_circuit* c, const pcb_evidence& ev, cudaStream_t st);
int32_t pcb_allreduce_range(pcb_circuit* c, uint64_t first, uint64_t count, cudaStream_t st);
int32_t pcb_dense_forward(pcb_circuit* c, pcb_workspace* ws, uint32_t layer, cudaStream_t st);
int32_t pcb_dense_backward(pcb_circuit* c, pcb_workspace* ws, uint32_t layer, cudaStream_t st);
// which of a workspace's per-set buffers a call needs: node matrices (klds / grads), the walk stacks of the
// one-warp-per-sample sampler, the relaxed sampler's per-edge matrices
enum { PCB_WS_NODES = 1, PCB_WS_STACK = 2, PCB_WS_EDGES = 4 };
int32_t pcb_ws_ensure_sets(pcb_workspace* ws, uint32_t S, int need);
int32_t pcb_dense_tc_forward(pcb_circuit* c, pcb_workspace* ws, uint32_t layer, cudaStream_t st);
int32_t pcb_dense_tc_backward(pcb_circuit* c, pcb_workspace* ws, uint32_t layer, cudaStream_t st);
int32_t pcb_check_status(pcb_circuit* c);
int32_t pcb_dense_tc_prepare(pcb_circuit* c, uint64_t* bytes);
int32_t pcb_dense_tc_refresh(pcb_circuit* c, cudaStream_t st);
int32_t pcb_side_join(pcb_circuit* c, cudaStream_t st);
int32_t pcb_dense_edge_prepare_ws(pcb_workspace* ws);
int32_t pcb_dense_edge_launch(pcb_circuit* c, pcb_workspace* ws, uint32_t o0, uint32_t n, uint32_t slices,
                              uint32_t b_per, cudaStream_t st);
int32_t pcb_dense_tc_flush_edges(pcb_circuit* c, pcb_workspace* ws, cudaStream_t st);
int32_t pcb_dense_mn_prepare(pcb_circuit* c, uint64_t* bytes);
int32_t pcb_dense_mn_refresh(pcb_circuit* c, cudaStream_t st);
int32_t pcb_dense_mn_forward(pcb_circuit* c, pcb_workspace* ws, uint32_t layer, cudaStream_t st);
int32_t pcb_dense_mn_backward_child(pcb_circuit* c, pcb_workspace* ws, uint32_t layer, cudaStream_t st);
