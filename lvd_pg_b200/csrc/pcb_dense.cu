// pcb_dense.cu — dense sum blocks (R parents over the same K children) as max-rescaled
// linear-domain matrix products.
//
// For a block with log-weights theta[r][t] and child values M[t][b] (= mars[c0+t][b] (+ mars[d0+t][b])):
//   mx[b]   = max_t M[t][b]                       A[t][b] = exp(M[t][b] - mx[b])
//   forward   mars[p0+r][b] = log(sum_t exp(theta[r][t]) * A[t][b]) + mx[b]
//   backward  G[r][b] = flows[p0+r][b] * exp(mx[b] - mars[p0+r][b])
//             flows[child t][b]  = A[t][b] * sum_r G[r][b] * exp(theta[r][t])
//             aggr[r][t]        += exp(theta[r][t]) * sum_b G[r][b] * A[t][b]
// which is the reference's per-edge arithmetic (queries/likelihood.jl:30-48, queries/flow.jl:53-81:
// edge flow = flows[parent] * exp(child + logp - mars[parent])) with one exp per node and example
// instead of one exp/log pair per edge and example.
//
// This file holds the fp32 SIMT version: shared-memory tiled, 4x4 register blocking.
#include <algorithm>

#include "pcb_internal.h"

namespace {

constexpr int TB = 128;  // examples per tile
constexpr int TR = 32;   // output rows per tile
constexpr int KC = 32;   // contraction chunk
constexpr int NT = 256;

__device__ __forceinline__ float child_val(const float* __restrict__ mars, uint32_t ld, const PcbDenseBlock& k,
                                           uint32_t t, uint32_t b) {
  float v = mars[(size_t)(k.c0 + t) * ld + b];
  if (k.d0 != PCB_NONE) v += mars[(size_t)(k.d0 + t) * ld + b];
  return v;
}

// grid: (ld / TB tiles, ceil(R / TR), blocks of the layer)
__global__ void __launch_bounds__(NT) dense_fwd_kernel(float* __restrict__ mars, float* __restrict__ blk_mx,
                                                       uint32_t ld, const PcbDenseBlock* __restrict__ blocks,
                                                       const float* __restrict__ theta) {
  __shared__ __align__(16) float As[KC][TB];
  __shared__ __align__(16) float Ws[KC][TR + 4];
  __shared__ float mxs[2][TB];
  const PcbDenseBlock k = blocks[blockIdx.z];
  const uint32_t r0 = blockIdx.y * TR;
  if (r0 >= k.R) return;
  const uint32_t b0 = blockIdx.x * TB;
  const uint32_t tid = threadIdx.x;
  const uint32_t tx = tid & 31, ty = tid >> 5;

  {  // per-example max over the K children
    uint32_t bl = tid & (TB - 1), half = tid >> 7;
    uint32_t b = b0 + bl;
    float mx = -INFINITY;
    if (b < ld)
      for (uint32_t t = half; t < k.K; t += 2) mx = fmaxf(mx, child_val(mars, ld, k, t, b));
    mxs[half][bl] = mx;
  }
  __syncthreads();
  if (tid < TB) {
    float mx = fmaxf(mxs[0][tid], mxs[1][tid]);
    mxs[0][tid] = mx;
    if (blockIdx.y == 0 && b0 + tid < ld) blk_mx[(size_t)k.mx_row * ld + b0 + tid] = mx;
  }
  __syncthreads();

  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.0f;

  for (uint32_t t0 = 0; t0 < k.K; t0 += KC) {
    {  // A chunk: exp(M - mx)
      uint32_t bl = tid & (TB - 1);
      uint32_t b = b0 + bl;
      float mx = mxs[0][bl];
#pragma unroll 4
      for (uint32_t q = 0; q < KC / 2; ++q) {
        uint32_t tl = (tid >> 7) + 2 * q, t = t0 + tl;
        float v = 0.0f;
        if (t < k.K && b < ld && mx != -INFINITY) v = __expf(child_val(mars, ld, k, t, b) - mx);
        As[tl][bl] = v;
      }
    }
    {  // W chunk: exp(theta[r][t]) stored [t][r]
      uint32_t tl = tid & 31, t = t0 + tl;
#pragma unroll
      for (uint32_t q = 0; q < TR / 8; ++q) {
        uint32_t rl = (tid >> 5) + 8 * q, r = r0 + rl;
        float w = 0.0f;
        if (t < k.K && r < k.R) w = __expf(__ldg(theta + k.pid0 + (size_t)r * k.K + t));
        Ws[tl][rl] = w;
      }
    }
    __syncthreads();
#pragma unroll 8
    for (int tl = 0; tl < KC; ++tl) {
      float4 a = *reinterpret_cast<const float4*>(&As[tl][tx * 4]);
      float4 w = *reinterpret_cast<const float4*>(&Ws[tl][ty * 4]);
      float av[4] = {a.x, a.y, a.z, a.w}, wv[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(wv[i], av[j], acc[i][j]);
    }
    __syncthreads();
  }
  uint32_t b = b0 + tx * 4;
  if (b < ld) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      uint32_t r = r0 + ty * 4 + i;
      if (r >= k.R) continue;
      float4 o;
      float* ov = reinterpret_cast<float*>(&o);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float mx = mxs[0][tx * 4 + j];
        ov[j] = mx == -INFINITY ? -INFINITY : __logf(acc[i][j]) + mx;
      }
      *reinterpret_cast<float4*>(&mars[(size_t)(k.p0 + r) * ld + b]) = o;
    }
  }
}

// flows of the K children.  grid: (ld / TB tiles, ceil(K / TR), blocks of the layer)
__global__ void __launch_bounds__(NT) dense_bwd_child_kernel(float* __restrict__ flows, const float* __restrict__ mars,
                                                             const float* __restrict__ blk_mx, uint32_t ld,
                                                             const PcbDenseBlock* __restrict__ blocks,
                                                             const float* __restrict__ theta) {
  __shared__ __align__(16) float Gs[KC][TB];
  __shared__ __align__(16) float Ws[KC][TR + 4];
  const PcbDenseBlock k = blocks[blockIdx.z];
  const uint32_t t0 = blockIdx.y * TR;
  if (t0 >= k.K) return;
  const uint32_t b0 = blockIdx.x * TB;
  const uint32_t tid = threadIdx.x;
  const uint32_t tx = tid & 31, ty = tid >> 5;
  const float* mxrow = blk_mx + (size_t)k.mx_row * ld;

  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.0f;

  for (uint32_t rc = 0; rc < k.R; rc += KC) {
    {
      uint32_t bl = tid & (TB - 1);
      uint32_t b = b0 + bl;
      float mx = b < ld ? mxrow[b] : -INFINITY;
#pragma unroll 4
      for (uint32_t q = 0; q < KC / 2; ++q) {
        uint32_t rl = (tid >> 7) + 2 * q, r = rc + rl;
        float g = 0.0f;
        if (r < k.R && b < ld && mx != -INFINITY) {
          size_t o = (size_t)(k.p0 + r) * ld + b;
          g = flows[o] * __expf(mx - mars[o]);
        }
        Gs[rl][bl] = g;
      }
    }
    {
      uint32_t tl = tid & 31, t = t0 + tl;
#pragma unroll
      for (uint32_t q = 0; q < KC / 8; ++q) {
        uint32_t rl = (tid >> 5) + 8 * q, r = rc + rl;
        float w = 0.0f;
        if (t < k.K && r < k.R) w = __expf(__ldg(theta + k.pid0 + (size_t)r * k.K + t));
        Ws[rl][tl] = w;
      }
    }
    __syncthreads();
#pragma unroll 8
    for (int rl = 0; rl < KC; ++rl) {
      float4 g = *reinterpret_cast<const float4*>(&Gs[rl][tx * 4]);
      float4 w = *reinterpret_cast<const float4*>(&Ws[rl][ty * 4]);
      float gv[4] = {g.x, g.y, g.z, g.w}, wv[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(wv[i], gv[j], acc[i][j]);
    }
    __syncthreads();
  }
  uint32_t b = b0 + tx * 4;
  if (b < ld) {
    float4 mx4 = *reinterpret_cast<const float4*>(&mxrow[b]);
    const float* mxv = reinterpret_cast<const float*>(&mx4);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      uint32_t t = t0 + ty * 4 + i;
      if (t >= k.K) continue;
      float4 o;
      float* ov = reinterpret_cast<float*>(&o);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float a = mxv[j] == -INFINITY ? 0.0f : __expf(child_val(mars, ld, k, t, b + j) - mxv[j]);
        ov[j] = acc[i][j] * a;
      }
      *reinterpret_cast<float4*>(&flows[(size_t)(k.c0 + t) * ld + b]) = o;
      if (k.d0 != PCB_NONE) *reinterpret_cast<float4*>(&flows[(size_t)(k.d0 + t) * ld + b]) = o;
    }
  }
}

// edge statistics.  64x64 tile of (r, t), contraction over a slice of the examples.
// grid: (B slices, ceil(R/64) * ceil(K/64), blocks of the layer)
constexpr int ER = 64, ET = 64, EB = 32;
__global__ void __launch_bounds__(NT) dense_bwd_edge_kernel(const float* __restrict__ flows, const float* __restrict__ mars,
                                                            const float* __restrict__ blk_mx, uint32_t ld, uint32_t B,
                                                            uint32_t b_per_cta, const PcbDenseBlock* __restrict__ blocks,
                                                            const float* __restrict__ theta, float* __restrict__ aggr) {
  __shared__ float Gs[ER][EB + 1];
  __shared__ float As[ET][EB + 1];
  const PcbDenseBlock k = blocks[blockIdx.z];
  const uint32_t tiles_t = (k.K + ET - 1) / ET;
  const uint32_t r0 = (blockIdx.y / tiles_t) * ER, t0 = (blockIdx.y % tiles_t) * ET;
  if (r0 >= k.R) return;
  const uint32_t tid = threadIdx.x;
  const uint32_t tx = tid & 15, ty = tid >> 4;
  const float* mxrow = blk_mx + (size_t)k.mx_row * ld;
  const uint32_t bs = blockIdx.x * b_per_cta, be = min(B, bs + b_per_cta);

  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.0f;

  for (uint32_t bc = bs; bc < be; bc += EB) {
    uint32_t bl = tid & 31;
    uint32_t b = bc + bl;
    bool bok = b < be;
    float mx = bok ? mxrow[b] : -INFINITY;
#pragma unroll 4
    for (uint32_t q = 0; q < ER / 8; ++q) {
      uint32_t rl = (tid >> 5) + 8 * q, r = r0 + rl;
      float g = 0.0f;
      if (bok && r < k.R && mx != -INFINITY) {
        size_t o = (size_t)(k.p0 + r) * ld + b;
        g = flows[o] * __expf(mx - mars[o]);
      }
      Gs[rl][bl] = g;
    }
#pragma unroll 4
    for (uint32_t q = 0; q < ET / 8; ++q) {
      uint32_t tl = (tid >> 5) + 8 * q, t = t0 + tl;
      float a = 0.0f;
      if (bok && t < k.K && mx != -INFINITY) a = __expf(child_val(mars, ld, k, t, b) - mx);
      As[tl][bl] = a;
    }
    __syncthreads();
#pragma unroll 8
    for (int x = 0; x < EB; ++x) {
      float gv[4], av[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) gv[i] = Gs[ty * 4 + i][x];
#pragma unroll
      for (int j = 0; j < 4; ++j) av[j] = As[tx * 4 + j][x];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(gv[i], av[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    uint32_t r = r0 + ty * 4 + i;
    if (r >= k.R) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      uint32_t t = t0 + tx * 4 + j;
      if (t >= k.K) continue;
      size_t p = k.pid0 + (size_t)r * k.K + t;
      atomicAdd(aggr + p, __expf(__ldg(theta + p)) * acc[i][j]);
    }
  }
}

}  // namespace

int32_t pcb_dense_forward(pcb_circuit* c, pcb_workspace* ws, uint32_t layer, cudaStream_t st) {
  if (c->use_tc) return pcb_dense_tc_forward(c, ws, layer, st);
  uint32_t o0 = c->h_dense_off[layer], o1 = c->h_dense_off[layer + 1];
  if (o1 == o0) return PCB_OK;
  uint32_t bt = (pcb_round_up(ws->B, 32) + TB - 1) / TB;
  dim3 grid(bt, (c->max_dense_R + TR - 1) / TR, o1 - o0);
  { PcbProfScope ps(c, st, PCB_K_DENSE_FWD); dense_fwd_kernel<<<grid, NT, 0, st>>>(ws->mars, ws->blk_mx, ws->ld, c->dense + o0, c->theta); }
  return PCB_OK;
}

int32_t pcb_dense_backward(pcb_circuit* c, pcb_workspace* ws, uint32_t layer, cudaStream_t st) {
  if (c->use_tc) return pcb_dense_tc_backward(c, ws, layer, st);
  uint32_t o0 = c->h_dense_off[layer], o1 = c->h_dense_off[layer + 1];
  if (o1 == o0) return PCB_OK;
  uint32_t bt = (pcb_round_up(ws->B, 32) + TB - 1) / TB;
  dim3 grid(bt, (c->max_dense_K + TR - 1) / TR, o1 - o0);
  { PcbProfScope ps(c, st, PCB_K_DENSE_BWD_CHILD); dense_bwd_child_kernel<<<grid, NT, 0, st>>>(ws->flows, ws->mars, ws->blk_mx, ws->ld, c->dense + o0, c->theta); }
  if (c->skip_stats) return PCB_OK;   // flows only
  uint32_t tiles = ((c->max_dense_R + ER - 1) / ER) * ((c->max_dense_K + ET - 1) / ET);
  // enough example slices to fill the GPU when the layer has few blocks
  uint32_t want = std::max(1u, (148u * 4u) / std::max(1u, tiles * (o1 - o0)));
  uint32_t slices = std::min(want, (ws->B + 127) / 128);
  uint32_t b_per = pcb_round_up((ws->B + slices - 1) / slices, EB);
  slices = (ws->B + b_per - 1) / b_per;
  dim3 egrid(slices, tiles, o1 - o0);
  { PcbProfScope ps(c, st, PCB_K_DENSE_BWD_EDGE); dense_bwd_edge_kernel<<<egrid, NT, 0, st>>>(ws->flows, ws->mars, ws->blk_mx, ws->ld, ws->B, b_per, c->dense + o0,
                                              c->theta, c->aggr); }
  return PCB_OK;
}
