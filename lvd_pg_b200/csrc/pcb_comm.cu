// pcb_comm.cu — the one collective of the multi-GPU EM step: a float sum all-reduce of the
// statistics vector [edge flows | leaf flow slots | batch log-likelihood] over NCCL.
//
// The reference has no multi-GPU data path (it runs independent jobs, one per GPU:
// exps/progressive_growing/pg.sh:2-7).  Here every rank holds a replica of the parameters,
// processes its shard of the batch, and after this all-reduce applies the identical update.
//
// NCCL is bound at run time with dlopen so that libpcb200.so loads on machines without it and so
// that a host process which already carries NCCL (PyTorch, CUDA.jl) shares the one copy.
#include <dlfcn.h>

#include <chrono>
#include <cstdlib>
#include <cstring>
#include <string>
#include <thread>

#include "pcb_internal.h"

namespace {

typedef struct { char internal[128]; } nccl_uid;
typedef int (*fn_get_uid)(nccl_uid*);
typedef int (*fn_init_rank)(void** comm, int nranks, nccl_uid id, int rank);
typedef int (*fn_allreduce)(const void*, void*, size_t, int dtype, int op, void* comm, cudaStream_t);
typedef int (*fn_destroy)(void* comm);
typedef int (*fn_async_error)(void* comm, int* async_error);
typedef const char* (*fn_errstr)(int);

struct NcclApi {
  void* handle = nullptr;
  fn_get_uid get_uid = nullptr;
  fn_init_rank init_rank = nullptr;
  fn_allreduce allreduce = nullptr;
  fn_destroy destroy = nullptr;
  fn_destroy abort = nullptr;
  fn_async_error async_error = nullptr;
  fn_errstr errstr = nullptr;
};
NcclApi g_nccl;

int32_t load_nccl() {
  if (g_nccl.handle) return PCB_OK;
  // PCB_NCCL_LIBRARY names the library to bind instead of the default sonames
  const char* names[] = {getenv("PCB_NCCL_LIBRARY"), "libnccl.so.2", "libnccl.so"};
  void* h = nullptr;
  for (const char* n : names) {
    if (!n || !*n) continue;
    h = dlopen(n, RTLD_NOW | RTLD_GLOBAL);
    if (h) break;
  }
  if (!h) return pcb_fail(PCB_ERR_NCCL, std::string("cannot load NCCL: ") + dlerror());
  g_nccl.get_uid = (fn_get_uid)dlsym(h, "ncclGetUniqueId");
  g_nccl.init_rank = (fn_init_rank)dlsym(h, "ncclCommInitRank");
  g_nccl.allreduce = (fn_allreduce)dlsym(h, "ncclAllReduce");
  g_nccl.destroy = (fn_destroy)dlsym(h, "ncclCommDestroy");
  g_nccl.abort = (fn_destroy)dlsym(h, "ncclCommAbort");
  g_nccl.async_error = (fn_async_error)dlsym(h, "ncclCommGetAsyncError");
  g_nccl.errstr = (fn_errstr)dlsym(h, "ncclGetErrorString");
  if (!g_nccl.get_uid || !g_nccl.init_rank || !g_nccl.allreduce || !g_nccl.destroy || !g_nccl.abort ||
      !g_nccl.async_error || !g_nccl.errstr)
    return pcb_fail(PCB_ERR_NCCL, "NCCL library lacks a required symbol");
  g_nccl.handle = h;
  return PCB_OK;
}

int32_t nccl_fail(const char* what, int code) {
  return pcb_fail(PCB_ERR_NCCL, std::string(what) + ": " + (g_nccl.errstr ? g_nccl.errstr(code) : "?"));
}

// Every captured step of the circuit holds a reference to its communicator; ncclCommDestroy (and
// the tear-down behind ncclCommAbort) waits until the last such graph is gone.  A graph that is
// still running is freed by the driver when it completes.
void drop_step_graphs(pcb_circuit* c) {
  std::lock_guard<std::mutex> g(c->ws_mu);
  for (pcb_workspace* ws : c->workspaces) {
    if (ws->step_exec) { cudaGraphExecDestroy(ws->step_exec); ws->step_exec = nullptr; }
    ws->have_key = false;
  }
}

}  // namespace

extern "C" int32_t pcb_comm_unique_id(uint8_t* id_out_128) {
  PCB_REQUIRE(id_out_128, "null argument");
  int32_t st = load_nccl();
  if (st != PCB_OK) return st;
  nccl_uid id;
  int rc = g_nccl.get_uid(&id);
  if (rc != 0) return nccl_fail("ncclGetUniqueId", rc);
  memcpy(id_out_128, id.internal, 128);
  return PCB_OK;
}

extern "C" int32_t pcb_comm_init(pcb_circuit* c, const uint8_t* id_128, int32_t rank, int32_t nranks) {
  PCB_REQUIRE(c && id_128, "null argument");
  PCB_REQUIRE(nranks >= 1 && rank >= 0 && rank < nranks, "bad rank / nranks");
  PCB_REQUIRE(c->comm == nullptr, "communicator already attached");
  int32_t st = load_nccl();
  if (st != PCB_OK) return st;
  PCB_CUDA(cudaSetDevice(c->device));
  nccl_uid id;
  memcpy(id.internal, id_128, 128);
  void* comm = nullptr;
  int rc = g_nccl.init_rank(&comm, nranks, id, rank);
  if (rc != 0) return nccl_fail("ncclCommInitRank", rc);
  c->comm = comm;
  c->rank = rank;
  c->nranks = nranks;
  c->comm_enabled = true;
  c->comm_lost = false;
  if (const char* e = getenv("PCB_COMM_SPLIT")) c->comm_split = atoi(e) != 0;
  if (const char* e = getenv("PCB_COMM_PIPE")) c->comm_pipe = atoi(e) != 0;
  if (!c->comm_stream) {
    PCB_CUDA(cudaStreamCreateWithFlags(&c->comm_stream, cudaStreamNonBlocking));
    for (cudaEvent_t* ev : {&c->ev_c0, &c->ev_c1, &c->ev_c2, &c->ev_c3})
      PCB_CUDA(cudaEventCreateWithFlags(ev, cudaEventDisableTiming));
  }
  return PCB_OK;
}

extern "C" int32_t pcb_comm_set_enabled(pcb_circuit* c, int32_t enabled) {
  PCB_REQUIRE(c, "null argument");
  c->comm_enabled = enabled != 0;
  return PCB_OK;
}

extern "C" int32_t pcb_comm_destroy(pcb_circuit* c) {
  PCB_REQUIRE(c, "null argument");
  if (c->comm && g_nccl.destroy) {
    cudaSetDevice(c->device);
    cudaDeviceSynchronize();
    drop_step_graphs(c);
    g_nccl.destroy(c->comm);
  }
  c->comm = nullptr;
  c->comm_lost = false;
  c->nranks = 1;
  c->rank = 0;
  return PCB_OK;
}

extern "C" int32_t pcb_comm_poll(pcb_circuit* c) {
  PCB_REQUIRE(c, "null argument");
  if (c->comm_lost) return pcb_fail(PCB_ERR_NCCL, "the communicator was aborted");
  if (!c->comm) return PCB_OK;
  int async = 0;
  int rc = g_nccl.async_error(c->comm, &async);
  if (rc != 0) return nccl_fail("ncclCommGetAsyncError", rc);
  if (async != 0) return nccl_fail("asynchronous NCCL error", async);
  return PCB_OK;
}

extern "C" int32_t pcb_comm_abort(pcb_circuit* c) {
  PCB_REQUIRE(c, "null argument");
  if (!c->comm) return PCB_OK;
  cudaSetDevice(c->device);
  // no device synchronisation here: the reason to abort is usually a collective that will not end
  drop_step_graphs(c);
  int rc = g_nccl.abort(c->comm);
  c->comm = nullptr;
  c->comm_lost = true;   // steps refuse to run until pcb_comm_destroy or a new pcb_comm_init
  if (rc != 0) return nccl_fail("ncclCommAbort", rc);
  return PCB_OK;
}

extern "C" int32_t pcb_comm_wait(pcb_circuit* c, pcb_stream s, uint32_t timeout_ms) {
  PCB_REQUIRE(c, "null argument");
  PCB_CUDA(cudaSetDevice(c->device));
  cudaStream_t st = (cudaStream_t)s;
  const auto t0 = std::chrono::steady_clock::now();
  for (;;) {
    cudaError_t q = cudaStreamQuery(st);
    if (q == cudaSuccess) return pcb_comm_poll(c);
    if (q != cudaErrorNotReady) return pcb_fail(PCB_ERR_CUDA, std::string("cudaStreamQuery: ") + cudaGetErrorString(q));
    int32_t rc = pcb_comm_poll(c);
    const bool late = std::chrono::steady_clock::now() - t0 > std::chrono::milliseconds(timeout_ms);
    if (rc != PCB_OK || late) {
      std::string why = rc != PCB_OK ? std::string(pcb_last_error()) : "the stream did not drain within " + std::to_string(timeout_ms) + " ms";
      pcb_comm_abort(c);
      return pcb_fail(PCB_ERR_NCCL, why + "; communicator aborted");
    }
    std::this_thread::sleep_for(std::chrono::microseconds(200));
  }
}

int32_t pcb_allreduce_range(pcb_circuit* c, uint64_t first, uint64_t count, cudaStream_t st) {
  if (c->comm_lost) return pcb_fail(PCB_ERR_STATE, "the communicator was aborted: pcb_comm_destroy, then attach a new one");
  if (!c->comm || c->nranks == 1 || !c->comm_enabled || count == 0) return PCB_OK;
  // ncclFloat32 = 7, ncclSum = 0 (nccl.h: ncclDataType_t / ncclRedOp_t)
  int rc = g_nccl.allreduce(c->aggr + first, c->aggr + first, (size_t)count, 7, 0, c->comm, st);
  if (rc != 0) return nccl_fail("ncclAllReduce", rc);
  return PCB_OK;
}

int32_t pcb_allreduce_aggr(pcb_circuit* c, cudaStream_t st) { return pcb_allreduce_range(c, 0, c->aggr_len, st); }
