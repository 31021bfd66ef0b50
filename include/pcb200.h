/* pcb200.h — C ABI of libpcb200.so: the probabilistic-circuit hot path of
 * LVD-PG / VariationalJuice.jl on NVIDIA B200 (sm_100a).
 *
 * Conventions
 *  - Every entry point returns an int32 status (PCB_OK == 0).  No C++ exception
 *    crosses the boundary; pcb_last_error() gives the message of the last
 *    failure on the calling thread.
 *  - Pointers named *_dev are device pointers on the circuit's GPU, everything
 *    else is host memory.  All device work is enqueued on the cudaStream_t given
 *    by the caller (pass 0 for the legacy default stream).
 *  - Node, edge, variable and row ids in the descriptor and in row_ids are
 *    1-based, exactly as the Julia side holds them; the conversion to 0-based
 *    happens once inside pcb_circuit_create.
 *  - Matrices are column-major with the example (or parameter-set) index
 *    fastest, i.e. element (b, n) of a [B, N] matrix lives at b + ld*n, which is
 *    the layout of the reference's CuMatrix buffers.
 *  - The library never falls back to the CPU.
 */
#ifndef PCB200_H
#define PCB200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum {
  PCB_OK = 0,
  PCB_ERR_INVALID = 1,   /* bad argument / malformed circuit            */
  PCB_ERR_CUDA = 2,      /* a CUDA runtime call failed                  */
  PCB_ERR_NCCL = 3,      /* NCCL missing or a collective failed         */
  PCB_ERR_TOO_LARGE = 4, /* exceeds a stated static limit               */
  PCB_ERR_STATE = 5      /* call order violated (e.g. backward first)   */
};

enum { PCB_INPUT = 0, PCB_PRODUCT = 1, PCB_SUM = 2 };

/* Edge tag bits, meaning fixed by their use in
 * VariationalJuice.jl/src/queries/likelihood.jl:23-27 and queries/flow.jl:38-47. */
enum {
  PCB_TAG_FIRST = 1,
  PCB_TAG_LAST = 2,
  PCB_TAG_PARTIAL = 4,
  PCB_TAG_ONLYSUB = 8,
  PCB_TAG_USER = 16
};

/* Flattened compiled circuit in the reference's order: the content of
 * BitsProbCircuit (fields used at VariationalJuice.jl/src/bits_circuit.jl:40-42,76-99
 * and regularization/reg_em.jl:171-174).  Nodes are ordered children-before-parent
 * with the root last; a parent's up-edges are contiguous; up-edges are grouped by
 * layer (up_layer_ends are 1-based inclusive ends); down-edges are described by
 * down2up (down-edge id -> up-edge id) and their own layer ends. */
typedef struct pcb_circuit_desc {
  uint32_t num_nodes;
  uint32_t num_edges;
  uint32_t num_up_layers;
  uint32_t num_down_layers;
  uint32_t num_input_nodes;
  uint32_t num_vars;
  uint64_t heap_len;
  const uint8_t* node_kind;        /* [N] PCB_INPUT / PCB_PRODUCT / PCB_SUM          */
  const uint32_t* node_var;        /* [N] variable of an input node, 0 otherwise      */
  const uint32_t* node_num_cats;   /* [N] categories of an input node                 */
  const uint32_t* node_heap_start; /* [N] 1-based heap index of the first log-prob    */
  const uint8_t* node_fixed;       /* [N] 1: input has no learnable parameters        */
  const uint32_t* up_parent;       /* [E]                                             */
  const uint32_t* up_prime;        /* [E]                                             */
  const uint32_t* up_sub;          /* [E] 0 when the edge has a single child          */
  const float* up_logp;            /* [E] log-parameter of a sum edge, 0 for products */
  const uint8_t* up_tag;           /* [E] PCB_TAG_* bits (may be NULL)                */
  const uint32_t* up_layer_ends;   /* [num_up_layers]                                 */
  const uint32_t* down2up;         /* [E]                                             */
  const uint32_t* down_layer_ends; /* [num_down_layers]                               */
  const uint32_t* input_node_ids;  /* [num_input_nodes]                               */
  const float* heap;               /* [heap_len] leaf storage, layout of
                                      nodes/fixable_categorical_dist.jl:54-64: C log-probs,
                                      then (learnable leaves only) C flow slots + 1 missing slot */
} pcb_circuit_desc;

typedef struct pcb_circuit pcb_circuit;     /* compiled circuit + parameters on one GPU */
typedef struct pcb_workspace pcb_workspace; /* mars / flows buffers for a max batch      */
typedef void* pcb_stream;                   /* cudaStream_t                              */

/* Counters of a compiled circuit (bits_circuit.jl:119-131 num_parameters, num_nodes,
 * num_edges, num_input_params, plus what the layout compiler found). */
typedef struct pcb_circuit_info {
  uint32_t num_nodes, num_edges, num_sum_edges, num_up_layers;
  uint32_t num_inner_params, num_input_params, num_param_groups;
  uint32_t num_dense_blocks, num_sum_regions, max_group_size, max_num_cats;
  uint64_t num_dense_edges;
  uint64_t device_bytes;
  uint32_t num_heads, reserved;
} pcb_circuit_info;

const char* pcb_last_error(void);
int32_t pcb_version(void);

/* ---- circuit ------------------------------------------------------------------------ */
/* Replaces cu(BitsProbCircuit) + CuMetaBitsProbCircuit(pc) (bits_circuit.jl:39-113):
 * uploads the circuit to `device`, builds the flat parameter maps and the packed layout. */
int32_t pcb_circuit_create(const pcb_circuit_desc* desc, int32_t device, pcb_circuit** out);
int32_t pcb_circuit_destroy(pcb_circuit* c);
int32_t pcb_circuit_get_info(const pcb_circuit* c, pcb_circuit_info* info);
/* Waits for the circuit's device and reports whether any kernel of this circuit gave up a bounded
 * wait since the circuit was created (PCB_ERR_CUDA; the statistics of that step are then
 * incomplete).  A training loop calls it where it synchronises anyway, e.g. when it reads the
 * epoch's log-likelihoods (the CUDA.synchronize() of regularization/reg_em.jl:288). */
int32_t pcb_circuit_status(pcb_circuit* c);

/* prep_memory(mars_mem / flows_mem, (batch_size, num_nodes)) of reg_em.jl:226-235.
 * `sets` != 0 additionally reserves the per-parameter-set buffers the KLD and
 * sampling calls need (klds, edge_klds, grads, ... of utils/cuda_preallocation.jl:6-45). */
int32_t pcb_workspace_create(pcb_circuit* c, uint32_t max_batch, int32_t sets, pcb_workspace** out);
int32_t pcb_workspace_destroy(pcb_workspace* ws);

/* ---- parameters --------------------------------------------------------------------- */
/* vectorize_parameters / update_parameters (misc.jl:5-68, 73-135): flat order = inner
 * (sum-edge) params in param2edge order, then leaf params in input_node_ids order. */
int32_t pcb_get_params(pcb_circuit* c, float* params_host, uint64_t n);
int32_t pcb_set_params(pcb_circuit* c, const float* params_host, uint64_t n);
int32_t pcb_get_params_dev(pcb_circuit* c, float* params_dev, uint64_t n, pcb_stream s);
int32_t pcb_set_params_dev(pcb_circuit* c, const float* params_dev, uint64_t n, pcb_stream s);
/* Copies of bpc.heap and of edge_aggr in down-edge order (conditional_pc/custom_em_tests.jl:88-90). */
int32_t pcb_get_heap(pcb_circuit* c, float* heap_host, uint64_t n);
int32_t pcb_get_edge_aggr(pcb_circuit* c, float* edge_aggr_host, uint64_t n);
/* Flat parameter maps of CuMetaBitsProbCircuit (bits_circuit.jl:44-70), 1-based. */
int32_t pcb_get_edge2param(pcb_circuit* c, uint32_t* edge2param_host, uint64_t n);
int32_t pcb_get_sum_regions(pcb_circuit* c, uint32_t* node_region_host, uint64_t n);

/* ---- forward / backward / EM -------------------------------------------------------- */
/* Forward pass: init_mar!_with_reg + layer_up over all layers
 * (regularization/reg_likelihood.jl:16-49,126-137, queries/likelihood.jl:4-113).
 * data_dev: [num_rows, num_vars] uint8 column-major; miss_dev: same shape, nonzero = missing
 * (may be NULL); row_ids_dev: B 1-based row ids (NULL => rows row_start .. row_start+B-1,
 * 1-based).  ll_out_dev (may be NULL) receives mars[1:B, end]. */
int32_t pcb_forward(pcb_circuit* c, pcb_workspace* ws, const uint8_t* data_dev,
                    const uint8_t* miss_dev, uint64_t num_rows, const int32_t* row_ids_dev,
                    uint32_t row_start, uint32_t B, float* ll_out_dev, pcb_stream s);
/* Backward pass of the batch last given to pcb_forward: reg_flows_circuit +
 * input_flows_circuit_with_reg (regularization/reg_flow.jl:24-48,120-274,
 * queries/flow.jl:8-159).  Adds to edge_aggr and to the leaf flow slots;
 * weights_dev (per data row, may be NULL) scales leaf flows only, as the reference does. */
int32_t pcb_backward(pcb_circuit* c, pcb_workspace* ws, const float* weights_dev, pcb_stream s);
/* edge_aggr .*= rate and clear_input_node_mem(bpc; rate) (reg_em.jl:276-284,
 * nodes/fixable_categorical_dist.jl:250-260). */
int32_t pcb_clear_flows(pcb_circuit* c, float rate, pcb_stream s);
/* add_pseudocount + aggr_node_flows + update_params + update_input_node_params
 * (reg_em.jl:292-299; arithmetic of pretrain/mini_batch_warmup.jl:4-76,
 * sgd/adam.jl:27-37, nodes/fixable_categorical_dist.jl:223-248). */
int32_t pcb_em_update(pcb_circuit* c, float pseudocount, float inertia, pcb_stream s);
/* One mini-batch step, the per-batch body of mini_batch_em_with_reg (reg_em.jl:273-301):
 * clear (rate), forward, backward, [all-reduce when a communicator is attached],
 * update.  ll_sum_dev receives sum(mars[1:B,end]) of the local shard. */
int32_t pcb_em_step(pcb_circuit* c, pcb_workspace* ws, const uint8_t* data_dev,
                    const uint8_t* miss_dev, uint64_t num_rows, const int32_t* row_ids_dev,
                    uint32_t row_start, uint32_t B, const float* weights_dev, float clear_rate,
                    float pseudocount, float inertia, float* ll_sum_dev, pcb_stream s);
/* What a batch is evaluated on, for the forms of the reference's passes that the plain entry
 * points above do not cover:
 *  - soft evidence (regularization/reg_likelihood.jl:51-91, reg_flow.jl:50-82): soft_dev holds a
 *    log-weight per (row, variable, category), [num_rows, num_vars, C] column-major, and takes the
 *    place of data_dev; a leaf's value is logsumexp_c(soft + logp_c), its statistics take
 *    exp(soft + logp_c - value) * flow per category;
 *  - soft-regularised leaves (soft_reg > 0 with hard evidence: reg_likelihood.jl:4-14, reg_flow.jl:3-22);
 *  - multi-head circuits (src-jl/multi_head_pc/): a circuit whose last node is a fake root sum whose
 *    edges carry PCB_TAG_USER; its children are the heads.  head_mask_dev [num_rows, num_heads]
 *    column-major gives every row's weight per head: root flows start from it (flow.jl:141-176) and
 *    the log-likelihood is logsumexp_h(value_h + log mask_h) - log sum_h mask_h (bit_circuit.jl:95-109).
 *    Without a mask only the forward pass is defined and ll_out_dev receives [B, num_heads]. */
typedef struct pcb_evidence {
  const uint8_t* data_dev;     /* [num_rows, num_vars] uint8 categories (NULL with soft_dev)   */
  const uint8_t* miss_dev;     /* same shape, nonzero = missing, may be NULL                   */
  const float* soft_dev;       /* per-category log-weights, or NULL                            */
  const float* head_mask_dev;  /* multi-head circuits only, may be NULL for the forward pass   */
  uint64_t num_rows;
  const int32_t* row_ids_dev;  /* B 1-based row ids, or NULL for rows row_start .. row_start+B-1 */
  uint32_t row_start, B;
  float soft_reg;              /* 0: plain lookup                                              */
  uint32_t soft_reg_width;
} pcb_evidence;
/* pcb_forward / pcb_em_step on such a batch (pcb_backward works on whatever the last forward saw);
 * multi_head_probs_flows_circuit / mini_batch_em_for_multihead_pc (src-jl/multi_head_pc/flow.jl:197-201,
 * em.jl:58-83) and the soft forms of mini_batch_em_with_reg are these calls in a loop. */
int32_t pcb_forward_ex(pcb_circuit* c, pcb_workspace* ws, const pcb_evidence* ev, float* ll_out_dev, pcb_stream s);
int32_t pcb_em_step_ex(pcb_circuit* c, pcb_workspace* ws, const pcb_evidence* ev, const float* weights_dev,
                       float clear_rate, float pseudocount, float inertia, float* ll_sum_dev, pcb_stream s);
/* per_sample_normalized_flows (queries/flow.jl:417-494): for every row of the batch, the flow of
 * every sum edge divided by the flow of its node, and of every leaf parameter by its leaf's, as
 * log(flow / (sum + 1e-8) + 1e-8) (map_flows_kernel :496-528) and log(flow / sum)
 * (map_input_flows_kernel :549-593), written to out_dev [num_rows, P] column-major at the row's data
 * index.  params_dev = NULL: the circuit's own parameters (the call runs the forward and backward
 * passes on the workspace; the statistics vector is not touched); else [num_rows, P] log-parameters, one vector
 * per data row (eval_circuit / flows_circuit with params, queries/likelihood.jl:119-302,
 * flow.jl:240-403).  Hard evidence without missing values, single-head circuits. */
int32_t pcb_normalized_flows(pcb_circuit* c, pcb_workspace* ws, const pcb_evidence* ev, const float* params_dev,
                             float* out_dev, pcb_stream s);
/* normalize_params(mbpc, params; undo) (misc.jl:363-392, 405-480) on [S, P] parameter sets, in place:
 * leaves become probabilities (exp, divided by the leaf's sum; undo: log(p + 1e-6) of the positive
 * entries), sum groups log-normalised (in both directions, as in the reference). */
int32_t pcb_normalize_params(pcb_circuit* c, float* params_dev, uint32_t S, int32_t undo, pcb_stream s);
/* map_pc_parameters_kernel (utils/map_params.jl:128-146): dst[s, ids_dst[i]] = src[s, ids_src[i]] for
 * i < n; both matrices have S rows (row index fastest), ids are 1-based parameter ids on the device.
 * The matching of two circuits' parameters (compute_mbpc_mapping) stays host code of the caller. */
int32_t pcb_map_param_columns(float* dst_dev, const float* src_dev, uint32_t S, const uint32_t* ids_dst_dev,
                              const uint32_t* ids_src_dev, uint32_t n, pcb_stream s);
/* Node ids (1-based) of the heads of a multi-head circuit, in head order. */
int32_t pcb_get_head_roots(pcb_circuit* c, uint32_t* roots_host, uint64_t n);

/* Parity accessors: mars / flows of the last batch, [B, num_nodes] column-major, ld = B. */
int32_t pcb_get_mars(pcb_circuit* c, pcb_workspace* ws, float* mars_host, uint64_t n);
int32_t pcb_get_flows(pcb_circuit* c, pcb_workspace* ws, float* flows_host, uint64_t n);

/* ---- KLD, its gradient, Adam -------------------------------------------------------- */
/* kld(mbpc, params1, params2) (queries/kld.jl:6-206): params are [S, P] column-major
 * log-parameters; kld_out_dev receives klds[1:S, end]. */
int32_t pcb_kld(pcb_circuit* c, pcb_workspace* ws, const float* params1_dev,
                const float* params2_dev, uint32_t S, float* kld_out_dev, pcb_stream s);
/* kld_backward (queries/kld.jl:212-320,471-577,593-649 + misc.jl:710-754) of the last pcb_kld
 * call: gradients w.r.t. the log-parameters, [S, P] column-major. */
int32_t pcb_kld_backward(pcb_circuit* c, pcb_workspace* ws, const float* params1_dev,
                         const float* params2_dev, uint32_t S, float* grads1_dev,
                         float* grads2_dev, pcb_stream s);
/* Parity accessors for the `reuse` tuple of kld() (queries/kld.jl:177-206): klds [S, N] of the
 * last pcb_kld call (host), and edge_klds [S, E] in up-edge order, which are not stored but
 * recomputed from the node values and the same two parameter matrices (device buffer). */
int32_t pcb_get_klds(pcb_circuit* c, pcb_workspace* ws, uint32_t S, float* klds_host);
int32_t pcb_kld_edge_klds(pcb_circuit* c, pcb_workspace* ws, const float* params1_dev,
                          const float* params2_dev, uint32_t S, float* edge_klds_dev, pcb_stream s);
/* Adam on a flat log-parameter vector followed by re-normalisation of every sum group and
 * every leaf (sgd/adam.jl:63-127,218-242).  sign = +1 ascends, -1 descends. */
int32_t pcb_adam_step(pcb_circuit* c, float* theta_dev, const float* grad_dev, float* m_dev,
                      float* v_dev, int32_t t, float lr, float beta1, float beta2, float eps,
                      float sign, pcb_stream s);

/* One step of the variational loop on a single parameter set: kld(q, p) (queries/kld.jl:164-206),
 * kld_backward with respect to q (:593-649), an Adam descent step on q's log-parameters and the
 * re-normalisation of every sum group and leaf (sgd/adam.jl:63-127,218-242) — what pcb_kld,
 * pcb_kld_backward and pcb_adam_step(sign = -1) do one after the other, as one call: a second call
 * with the same pointers and hyper-parameters captures the chain of launches as a CUDA graph and later
 * calls replay it (t must grow by one per call; any other value re-seeds the count).  theta_q_dev
 * [P] is updated in place; kld_out_dev (may be NULL) receives the KLD before the update. */
int32_t pcb_kld_adam_step(pcb_circuit* c, pcb_workspace* ws, float* theta_q_dev, const float* theta_p_dev,
                          float* m_dev, float* v_dev, int32_t t, float lr, float beta1, float beta2,
                          float eps, float* kld_out_dev, pcb_stream s);

/* ---- sampling ----------------------------------------------------------------------- */
/* Hard Gumbel-max top-down sampling, the temperature -> 0 limit of
 * queries/sample.jl:8-148,233-296 with caller-supplied uniforms.
 * params_dev: [Sp, P] column-major with Sp == 1 (shared) or Sp == S.
 * u_sum_dev: [S][num_sum_regions][max_group_size] uniforms (last index fastest);
 * u_leaf_dev: [S][num_vars][max_num_cats]; x_out_dev: [S, num_vars] column-major int32
 * 0-based categories; -1 for variables the walk did not reach. */
int32_t pcb_sample_hard(pcb_circuit* c, pcb_workspace* ws, const float* params_dev, uint32_t Sp,
                        const float* u_sum_dev, const float* u_leaf_dev, uint32_t S,
                        int32_t* x_out_dev, pcb_stream s);
/* Same samples as pcb_sample_hard, for callers that must not see this library allocate: no
 * workspace argument, no cudaMalloc / cudaFree inside.  Julia's CUDA.jl (and any host that has
 * given all device memory to its own pool) can be refused memory by a foreign cudaMalloc, which
 * also synchronises the device under its streams.  The walk stacks live in a static 4 MiB
 * device array of the library instead, so S * (num_vars + 2) must not exceed 2^20 words
 * (PCB_ERR_TOO_LARGE otherwise).  The array is shared: calls that overlap on the GPU race.  The
 * first call on a device looks the array's address up.  Every call waits for the stream before it
 * returns (it reads the walk's status word back), so it must not be made while the stream is
 * being captured.  This entry point has no counterpart in the reference. */
int32_t pcb_sample_hard_static(pcb_circuit* c, const float* params_dev, uint32_t Sp,
                               const float* u_sum_dev, const float* u_leaf_dev, uint32_t S,
                               int32_t* x_out_dev, pcb_stream s);
/* Soft Gumbel-softmax sampling (queries/sample.jl:8-383): u_dev [S, num_inner_params]
 * column-major uniforms or NULL for no_gumbel=true; out_dev is input_aggr_params
 * [S, num_vars, max_num_cats] column-major. */
int32_t pcb_sample_soft(pcb_circuit* c, pcb_workspace* ws, const float* params_dev, uint32_t Sp,
                        const float* u_dev, float temperature, uint32_t S, float* out_dev,
                        pcb_stream s);

/* conditioned_td_prob(mbpc, marked_pc_idx1, marked_pc_idx2, node_probs, input_aggr_params)
 * (queries/td_prob.jl:161-291): top-down probabilities with the circuit's own weights in which
 * inner node n with marked_var[n] > 0 takes node_probs[s, marked_var[n], marked_cat[n]] (1-based,
 * node_probs [S, Z1, Z2] column-major) instead of what its parents send; the leaves spread theirs
 * over their categories into out_dev [S, num_vars, max_num_cats] (zeroed by the call).
 * marked_*_dev: [num_nodes] int32 on the device. */
int32_t pcb_cond_td_prob(pcb_circuit* c, pcb_workspace* ws, const int32_t* marked_var_dev,
                         const int32_t* marked_cat_dev, const float* node_probs_dev, uint32_t S, uint32_t Z1,
                         float* out_dev, pcb_stream s);

/* ---- structure learning input ------------------------------------------------------------ */
/* pairwise_MI_chunked (utils/information.jl:3-157): mutual information of every pair of the
 * num_vars categorical columns of data_dev ([num_rows, num_vars] uint8, column-major, values below
 * num_cats, a power of two up to 256), with the pseudocount spread over the joint and the single
 * tables as the reference does; mi_dev [num_vars, num_vars] (symmetric).  No circuit is involved:
 * the call runs on the current device, allocates its scratch itself and returns when the result is
 * there. */
int32_t pcb_pairwise_mi(const uint8_t* data_dev, uint64_t num_rows, uint32_t num_vars, uint32_t num_cats,
                        float pseudocount, float* mi_dev, pcb_stream s);

/* ---- multi-GPU ---------------------------------------------------------------------- */
/* One NCCL communicator per process; pcb_em_step then sums [edge_aggr | leaf flows | LL]
 * over ranks before the replicated update.  The reference has no counterpart (it runs one
 * independent job per GPU, exps/progressive_growing/pg.sh:2-7). */
int32_t pcb_comm_unique_id(uint8_t* id_out_128);
int32_t pcb_comm_init(pcb_circuit* c, const uint8_t* id_128, int32_t rank, int32_t nranks);
int32_t pcb_comm_destroy(pcb_circuit* c);
/* enabled = 0: pcb_em_step skips its collectives although a communicator is attached (every rank then
 * updates from its own statistics).  For measuring how much of a step the communication leaves
 * exposed; not for training. */
int32_t pcb_comm_set_enabled(pcb_circuit* c, int32_t enabled);
/* Failure handling of the collective, all on the host; none of these waits on the device without a
 * limit.  pcb_comm_poll asks NCCL for an asynchronous error of the communicator (a peer that died,
 * a network fault) and returns PCB_ERR_NCCL with its text.  pcb_comm_wait is the bounded
 * counterpart of a stream synchronisation: it polls the stream `s` and the communicator every
 * 200 us until the stream has drained (PCB_OK), and on an asynchronous error or after timeout_ms
 * it aborts the communicator and returns PCB_ERR_NCCL.  pcb_comm_abort ends the communicator
 * without waiting for its collectives (ncclCommAbort: a collective in flight returns early, its
 * output is undefined); afterwards pcb_em_step returns PCB_ERR_STATE until pcb_comm_destroy has been
 * called, after which the circuit trains alone or takes a new communicator.  A training loop that
 * wants ranks to learn of a lost peer BEFORE they launch the next collective keeps a heartbeat on
 * the host (the Python mirror's RankWatch). */
int32_t pcb_comm_poll(pcb_circuit* c);
int32_t pcb_comm_wait(pcb_circuit* c, pcb_stream s, uint32_t timeout_ms);
int32_t pcb_comm_abort(pcb_circuit* c);

/* ---- launch accounting ---------------------------------------------------------------- */
/* The library counts its kernel launches per kernel class; with profiling enabled every launch
 * is also bracketed by two CUDA events on the caller's stream.  pcb_profile_read synchronises the
 * device and returns, per class, the summed event time in milliseconds and the launch count
 * (arrays of pcb_profile_num_classes() entries; either may be NULL); reset != 0 clears both.
 * The reference's counterpart is its debug=true path, which wraps each launch in CUDA.@time
 * (queries/likelihood.jl:86-92). */
int32_t pcb_profile_num_classes(void);
const char* pcb_profile_class_name(int32_t i);
int32_t pcb_profile_enable(pcb_circuit* c, int32_t on);
int32_t pcb_profile_read(pcb_circuit* c, double* ms_out, uint64_t* launches_out, int32_t reset);

/* ---- self-test of the bounded device waits ----------------------------------------------- */
/* Every mbarrier wait of the tensor-core kernels gives up after a fixed number of polls, raises the
 * circuit's status word (pcb_circuit_status) and lets the kernel drain and return.  This call runs
 * that wait on `device` on a barrier that nothing arrives at, limited to `polls` polls (at most 2^20):
 * *status_out = 1 (the word a circuit would report), *after_out = 2 (the kernel went on past the
 * lost wait and returned), *ms_out = the kernel's duration, *production_polls_out (may be NULL) =
 * the limit the production kernels use, so ms * production_polls / polls is how long a lost signal
 * holds a kernel.  The context stays usable.  No counterpart in the reference. */
int32_t pcb_selftest_wait_limit(int32_t device, uint32_t polls, int32_t* status_out, int32_t* after_out,
                                float* ms_out, uint32_t* production_polls_out);

/* ---- diagnostics -------------------------------------------------------------------------- */
/* Only in a library built with -DPCB_DIAG and with PCB_TC_TRACE set in the environment, CTA (0,0,0)
 * of every tensor-core dense kernel writes %globaltimer stamps of its pipeline events into a
 * 512-word device buffer; these calls synchronise the device and copy the buffer of the last traced
 * launch (forward / child-flow kernels, or the edge-statistics kernel) to `out` (512 words).
 * PCB_ERR_STATE when tracing is off, which it always is in the default build.  No counterpart in
 * the reference. */
int32_t pcb_debug_read_trace(unsigned long long* out);
int32_t pcb_debug_read_edge_trace(unsigned long long* out);

#ifdef __cplusplus
}
#endif
#endif /* PCB200_H */
