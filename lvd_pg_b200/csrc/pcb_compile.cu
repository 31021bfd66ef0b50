// pcb_compile.cu — circuit upload, layout compiler, parameter accessors, workspace.
//
// Replaces cu(BitsProbCircuit) + CuMetaBitsProbCircuit(pc)
// (VariationalJuice.jl/src/bits_circuit.jl:39-113) and vectorize/update_parameters
// (src/misc.jl:5-135).
#include <algorithm>
#include <cstdlib>
#include <cstring>
#include <unordered_map>

#include "../../include/pcb200_gumbel.h"
#include "pcb_internal.h"

static thread_local std::string g_last_error;

void pcb_set_error(const std::string& msg) { g_last_error = msg; }
int32_t pcb_fail(int32_t code, const std::string& msg) {
  g_last_error = msg;
  return code;
}

extern "C" const char* pcb_last_error(void) { return g_last_error.c_str(); }
extern "C" int32_t pcb_version(void) { return 100; }

namespace {

template <typename T>
int32_t upload(T** dst, const std::vector<T>& src, uint64_t* bytes) {
  size_t n = src.size() ? src.size() : 1;
  PCB_CUDA(cudaMalloc((void**)dst, n * sizeof(T)));
  if (src.size()) PCB_CUDA(cudaMemcpy(*dst, src.data(), src.size() * sizeof(T), cudaMemcpyHostToDevice));
  *bytes += n * sizeof(T);
  return PCB_OK;
}

#define PCB_TRY(expr)                  \
  do {                                 \
    int32_t _s = (expr);               \
    if (_s != PCB_OK) return _s;       \
  } while (0)

int32_t compile(const pcb_circuit_desc* d, pcb_circuit* c) {
  const uint32_t N = d->num_nodes, E = d->num_edges;
  PCB_REQUIRE(N >= 1, "circuit has no nodes");
  PCB_REQUIRE(d->node_kind && d->node_var && d->node_num_cats && d->node_heap_start && d->node_fixed,
              "node arrays missing");
  PCB_REQUIRE(E == 0 || (d->up_parent && d->up_prime && d->up_sub && d->up_logp && d->up_layer_ends && d->down2up),
              "edge arrays missing");
  PCB_REQUIRE(d->input_node_ids || d->num_input_nodes == 0, "input_node_ids missing");
  c->N = N; c->E = E; c->V = d->num_vars; c->L = d->num_up_layers;
  c->heap_len = d->heap_len;

  // ---- node edge ranges and layers -----------------------------------------------------
  std::vector<uint32_t> estart(N, 0), ecount(N, 0), layer(N, 0);
  std::vector<uint8_t> kind(d->node_kind, d->node_kind + N);
  {
    uint32_t lay = 1, e = 0;
    for (uint32_t li = 0; li < d->num_up_layers; ++li) {
      uint32_t end = d->up_layer_ends[li];
      PCB_REQUIRE(end <= E && end >= e, "up_layer_ends not increasing");
      for (; e < end; ++e) {
        uint32_t p = d->up_parent[e], pr = d->up_prime[e], sb = d->up_sub[e];
        PCB_REQUIRE(p >= 1 && p <= N && pr >= 1 && pr <= N && sb <= N, "edge endpoint out of range");
        --p; --pr;
        PCB_REQUIRE(kind[p] != PCB_INPUT, "an input node has an edge");
        if (ecount[p] == 0) { estart[p] = e; layer[p] = lay; }
        else PCB_REQUIRE(estart[p] + ecount[p] == e, "edges of a node are not contiguous");
        PCB_REQUIRE(layer[p] == lay, "edges of a node span several layers");
        ++ecount[p];
        PCB_REQUIRE(pr < p && (sb == 0 || sb - 1 < p), "children must precede their parent");
        PCB_REQUIRE(layer[pr] < lay && (sb == 0 || layer[sb - 1] < lay), "child not in an earlier layer");
        if (kind[pr] != PCB_INPUT) PCB_REQUIRE(ecount[pr] > 0, "child inner node has no edges yet");
      }
      ++lay;
    }
    PCB_REQUIRE(e == E, "up_layer_ends does not cover all edges");
  }

  // ---- parameter ids --------------------------------------------------------------------
  std::vector<uint32_t> e2p(E, PCB_NONE), n_pid0(N, PCB_NONE), grp_node;
  c->h_edge2param.assign(E, 0);
  uint32_t pid = 0;
  for (uint32_t e = 0; e < E; ++e) {
    uint32_t p = d->up_parent[e] - 1;
    if (kind[p] == PCB_SUM) {
      if (e == estart[p]) { n_pid0[p] = pid; grp_node.push_back(p); c->max_group = std::max(c->max_group, ecount[p]); }
      e2p[e] = pid;
      c->h_edge2param[e] = pid + 1;
      ++pid;
    }
  }
  c->n_inner = pid;
  c->n_groups = (uint32_t)grp_node.size();

  // ---- inputs ---------------------------------------------------------------------------
  const uint32_t NI = d->num_input_nodes;
  c->n_inputs = NI;
  std::vector<uint32_t> in_node(NI), in_var(NI), in_cats(NI), node2input(N, PCB_NONE);
  std::vector<uint64_t> in_poff(NI), in_foff(NI);
  c->h_in_fixed.resize(NI); c->h_heap_start.resize(NI);
  uint64_t lp = 0, fp = 0, fixed_p = 0;
  for (uint32_t i = 0; i < NI; ++i) {
    uint32_t n = d->input_node_ids[i];
    PCB_REQUIRE(n >= 1 && n <= N && kind[n - 1] == PCB_INPUT, "input_node_ids entry is not an input node");
    --n;
    PCB_REQUIRE(node2input[n] == PCB_NONE, "duplicate input node id");
    node2input[n] = i;
    in_node[i] = n;
    PCB_REQUIRE(d->node_var[n] >= 1 && d->node_var[n] <= d->num_vars, "leaf variable out of range");
    in_var[i] = d->node_var[n] - 1;
    in_cats[i] = d->node_num_cats[n];
    PCB_REQUIRE(in_cats[i] >= 1, "leaf without categories");
    c->max_cats = std::max(c->max_cats, in_cats[i]);
    c->h_in_fixed[i] = d->node_fixed[n];
    c->h_heap_start[i] = d->node_heap_start[n] - 1;
    uint64_t need = (uint64_t)c->h_heap_start[i] + in_cats[i] + (d->node_fixed[n] ? 0 : in_cats[i] + 1);
    PCB_REQUIRE(d->node_heap_start[n] >= 1 && need <= d->heap_len, "leaf heap slice out of range");
    if (!d->node_fixed[n]) { lp += in_cats[i]; }
  }
  for (uint32_t n = 0; n < N; ++n)
    if (kind[n] == PCB_INPUT) PCB_REQUIRE(node2input[n] != PCB_NONE, "input node missing from input_node_ids");
  c->n_input_params = (uint32_t)lp;
  c->P = (uint64_t)c->n_inner + lp;
  lp = 0;
  for (uint32_t i = 0; i < NI; ++i) {
    if (!c->h_in_fixed[i]) {
      in_poff[i] = c->n_inner + lp; lp += in_cats[i];
      in_foff[i] = c->n_inner + fp; fp += in_cats[i] + 1;
    } else {
      in_poff[i] = c->P + fixed_p; fixed_p += in_cats[i];
      in_foff[i] = ~0ull;
    }
  }
  c->theta_len = c->P + fixed_p;
  c->n_leaf_flow = fp;
  c->aggr_len = (uint64_t)c->n_inner + fp + 1;
  c->h_in_node = in_node; c->h_in_cats = in_cats; c->h_in_poff = in_poff; c->h_in_foff = in_foff;

  std::vector<float> theta(c->theta_len ? c->theta_len : 1, 0.0f);
  for (uint32_t e = 0; e < E; ++e) if (e2p[e] != PCB_NONE) theta[e2p[e]] = d->up_logp[e];
  for (uint32_t i = 0; i < NI; ++i)
    for (uint32_t k = 0; k < in_cats[i]; ++k) theta[in_poff[i] + k] = d->heap[c->h_heap_start[i] + k];

  // ---- down-edge permutation (kept for the edge_aggr accessor) ----------------------------
  c->h_down2up.resize(E);
  {
    std::vector<uint8_t> seen(E, 0);
    for (uint32_t de = 0; de < E; ++de) {
      uint32_t ue = d->down2up[de];
      PCB_REQUIRE(ue >= 1 && ue <= E && !seen[ue - 1], "down2up is not a permutation");
      seen[ue - 1] = 1;
      c->h_down2up[de] = ue - 1;
    }
  }

  // ---- sum regions (same rule as the oracle: scope signatures add over products) ----------
  std::vector<uint32_t> region(N, PCB_NONE);
  c->h_region1.assign(N, 0);
  {
    std::vector<uint64_t> sig(N, 0);
    std::vector<uint8_t> seen(N, 0);
    for (uint32_t n = 0; n < N; ++n)
      if (kind[n] == PCB_INPUT) { sig[n] = pcb_scope_mix(d->node_var[n]); seen[n] = 1; }
    for (uint32_t e = 0; e < E; ++e) {
      uint32_t p = d->up_parent[e] - 1;
      uint64_t cs = sig[d->up_prime[e] - 1] + (d->up_sub[e] ? sig[d->up_sub[e] - 1] : 0);
      if (kind[p] == PCB_PRODUCT) sig[p] += cs;
      else if (!seen[p]) { sig[p] = cs; seen[p] = 1; }
    }
    std::unordered_map<uint64_t, uint32_t> ids;
    for (uint32_t n = 0; n < N; ++n) {
      if (kind[n] != PCB_SUM) continue;
      uint64_t k = sig[n] | 1ull;
      auto it = ids.find(k);
      uint32_t r;
      if (it == ids.end()) { r = (uint32_t)ids.size(); ids.emplace(k, r); } else r = it->second;
      region[n] = r;
      c->h_region1[n] = r + 1;
    }
    c->n_regions = (uint32_t)ids.size();
  }

  // ---- multi-head circuits: the edges of the last node (a fake root over the heads) that carry the
  // user tag are skipped by every top-down pass (src-jl/multi_head_pc/bit_circuit.jl:22-34,
  // flow.jl:45); their prime children, in edge order, are the heads (root_ids of bit_circuit.jl:36-50)
  auto skipped = [&](uint32_t e) {
    return d->up_tag && (d->up_tag[e] & PCB_TAG_USER) && d->up_parent[e] == N;
  };
  std::vector<uint32_t> node_head(N, PCB_NONE);
  c->h_head_roots.clear();
  for (uint32_t e = 0; e < E; ++e)
    if (skipped(e)) {
      PCB_REQUIRE(d->up_sub[e] == 0, "a skipped fake-root edge must have a single child");
      node_head[d->up_prime[e] - 1] = (uint32_t)c->h_head_roots.size();
      c->h_head_roots.push_back(d->up_prime[e] - 1);
    }
  c->n_heads = (uint32_t)c->h_head_roots.size();

  // ---- CSR by child ---------------------------------------------------------------------
  std::vector<uint32_t> in_off(N + 1, 0);
  for (uint32_t e = 0; e < E; ++e) {
    if (skipped(e)) continue;
    ++in_off[d->up_prime[e]];            // (prime-1)+1
    if (d->up_sub[e]) ++in_off[d->up_sub[e]];
  }
  for (uint32_t n = 0; n < N; ++n) in_off[n + 1] += in_off[n];
  std::vector<PcbInEntry> in_ent(in_off[N] ? in_off[N] : 1);
  {
    std::vector<uint32_t> cur(in_off.begin(), in_off.end() - 1);
    for (uint32_t e = 0; e < E; ++e) {
      if (skipped(e)) continue;
      uint32_t p = d->up_parent[e] - 1, pr = d->up_prime[e] - 1;
      uint32_t sb = d->up_sub[e] ? d->up_sub[e] - 1 : PCB_NONE;
      in_ent[cur[pr]++] = PcbInEntry{p, sb, e2p[e], 1u};
      if (sb != PCB_NONE) in_ent[cur[sb]++] = PcbInEntry{p, pr, e2p[e], 0u};
    }
  }

  // ---- dense blocks -----------------------------------------------------------------------
  const bool allow_dense = !(getenv("PCB_DISABLE_DENSE") && atoi(getenv("PCB_DISABLE_DENSE")) != 0);
  const uint32_t MIN_K = 16, MIN_R = 16;
  std::vector<std::vector<uint32_t>> layer_nodes(c->L + 1);
  for (uint32_t e = 0; e < E; ++e) {
    uint32_t p = d->up_parent[e] - 1;
    if (e == estart[p]) layer_nodes[layer[p]].push_back(p);
  }
  for (uint32_t n = 0; n < N; ++n) if (kind[n] == PCB_INPUT || ecount[n] == 0) { layer[n] = 0; }
  std::vector<uint8_t> in_dense(N, 0), dense_child(N, 0);
  c->h_dense.clear();
  c->h_dense_off.assign(c->L + 2, 0);
  auto indeg = [&](uint32_t n) { return in_off[n + 1] - in_off[n]; };
  for (uint32_t lay = 1; lay <= c->L; ++lay) {
    c->h_dense_off[lay] = (uint32_t)c->h_dense.size();
    auto& ln = layer_nodes[lay];
    size_t i = 0;
    while (allow_dense && i < ln.size()) {
      uint32_t n = ln[i];
      uint32_t K = ecount[n];
      bool ok = kind[n] == PCB_SUM && K >= MIN_K;
      uint32_t c0 = 0, d0 = PCB_NONE;
      if (ok) {
        uint32_t e0 = estart[n];
        c0 = d->up_prime[e0] - 1;
        d0 = d->up_sub[e0] ? d->up_sub[e0] - 1 : PCB_NONE;
        for (uint32_t j = 0; j < K && ok; ++j) {
          ok = (d->up_prime[e0 + j] - 1 == c0 + j) &&
               (d0 == PCB_NONE ? d->up_sub[e0 + j] == 0 : d->up_sub[e0 + j] == d0 + j + 1);
        }
        if (ok && d0 != PCB_NONE) ok = (d0 >= c0 + K) || (c0 >= d0 + K);
      }
      if (!ok) { ++i; continue; }
      // extend the run over consecutive nodes with identical child lists
      size_t j = i + 1;
      while (j < ln.size()) {
        uint32_t m = ln[j];
        if (m != ln[j - 1] + 1 || kind[m] != PCB_SUM || ecount[m] != K || estart[m] != estart[ln[j - 1]] + K) break;
        if (memcmp(d->up_prime + estart[m], d->up_prime + estart[n], K * sizeof(uint32_t)) != 0) break;
        if (memcmp(d->up_sub + estart[m], d->up_sub + estart[n], K * sizeof(uint32_t)) != 0) break;
        ++j;
      }
      uint32_t R = (uint32_t)(j - i);
      bool excl = R >= MIN_R;
      for (uint32_t t = 0; t < K && excl; ++t) {
        excl = indeg(c0 + t) == R && !dense_child[c0 + t];
        if (excl && d0 != PCB_NONE) excl = indeg(d0 + t) == R && !dense_child[d0 + t];
      }
      if (!excl) { i = j; continue; }
      PcbDenseBlock blk{n, R, K, c0, d0, n_pid0[n], (uint32_t)c->h_dense.size(), 0};
      c->h_dense.push_back(blk);
      for (uint32_t r = 0; r < R; ++r) in_dense[n + r] = 1;
      for (uint32_t t = 0; t < K; ++t) { dense_child[c0 + t] = 1; if (d0 != PCB_NONE) dense_child[d0 + t] = 1; }
      c->dense_edges += (uint64_t)R * K;
      c->max_dense_K = std::max(c->max_dense_K, K);
      c->max_dense_R = std::max(c->max_dense_R, R);
      i = j;
    }
  }
  c->h_dense_off[c->L + 1] = (uint32_t)c->h_dense.size();
  c->n_dense = (uint32_t)c->h_dense.size();

  // ---- layer lists --------------------------------------------------------------------------
  std::vector<uint32_t> up_all, up_sparse, down_all, down_sparse;
  c->h_up_all_off.assign(c->L + 1, 0); c->h_up_sparse_off.assign(c->L + 1, 0);
  for (uint32_t lay = 1; lay <= c->L; ++lay) {
    c->h_up_all_off[lay - 1] = (uint32_t)up_all.size();
    c->h_up_sparse_off[lay - 1] = (uint32_t)up_sparse.size();
    for (uint32_t n : layer_nodes[lay]) { up_all.push_back(n); if (!in_dense[n]) up_sparse.push_back(n); }
  }
  c->h_up_all_off[c->L] = (uint32_t)up_all.size();
  c->h_up_sparse_off[c->L] = (uint32_t)up_sparse.size();
  // Chunks of eight consecutive nodes of a layer list whose edges lead to the same children in the
  // same order (the k sums of one HCLT variable do): a top-down pass that pushes to the children
  // adds the eight contributions in shared memory first.
  std::vector<uint8_t> up_same;
  c->h_up_chunk_off.assign(c->L + 1, 0);
  for (uint32_t lay = 1; lay <= c->L; ++lay) {
    c->h_up_chunk_off[lay - 1] = (uint32_t)up_same.size();
    const uint32_t o0 = c->h_up_all_off[lay - 1], o1 = c->h_up_all_off[lay];
    for (uint32_t b = o0; b < o1; b += 8) {
      const uint32_t first = up_all[b];
      bool same = kind[first] == PCB_SUM && ecount[first] <= 256;
      for (uint32_t i = b + 1; same && i < std::min(o1, b + 8); ++i) {
        const uint32_t n = up_all[i];
        same = kind[n] == PCB_SUM && ecount[n] == ecount[first] &&
               !memcmp(&d->up_prime[estart[n]], &d->up_prime[estart[first]], ecount[n] * sizeof(uint32_t)) &&
               !memcmp(&d->up_sub[estart[n]], &d->up_sub[estart[first]], ecount[n] * sizeof(uint32_t));
      }
      up_same.push_back(same ? 1 : 0);
    }
  }
  c->h_up_chunk_off[c->L] = (uint32_t)up_same.size();
  if (up_same.empty()) up_same.push_back(0);
  std::vector<std::vector<uint32_t>> by_layer(c->L + 1);
  for (uint32_t n = 0; n < N; ++n) by_layer[layer[n]].push_back(n);
  c->h_down_all_off.assign(c->L + 2, 0); c->h_down_sparse_off.assign(c->L + 2, 0);
  for (uint32_t lay = 0; lay <= c->L; ++lay) {
    c->h_down_all_off[lay] = (uint32_t)down_all.size();
    c->h_down_sparse_off[lay] = (uint32_t)down_sparse.size();
    for (uint32_t n : by_layer[lay]) { down_all.push_back(n); if (!dense_child[n]) down_sparse.push_back(n); }
  }
  c->h_down_all_off[c->L + 1] = (uint32_t)down_all.size();
  c->h_down_sparse_off[c->L + 1] = (uint32_t)down_sparse.size();

  // ---- upload ---------------------------------------------------------------------------------
  std::vector<uint32_t> e_prime(E), e_sub(E);
  for (uint32_t e = 0; e < E; ++e) { e_prime[e] = d->up_prime[e] - 1; e_sub[e] = d->up_sub[e] ? d->up_sub[e] - 1 : PCB_NONE; }
  uint64_t bytes = 0;
  PCB_TRY(upload(&c->theta, theta, &bytes));
  std::vector<float> aggr0(c->aggr_len, 0.0f);
  PCB_TRY(upload(&c->aggr, aggr0, &bytes));
  PCB_TRY(upload(&c->kind, kind, &bytes));
  PCB_TRY(upload(&c->n_estart, estart, &bytes));
  PCB_TRY(upload(&c->n_ecount, ecount, &bytes));
  PCB_TRY(upload(&c->n_pid0, n_pid0, &bytes));
  PCB_TRY(upload(&c->n_region, region, &bytes));
  {
    std::vector<uint4> sn(N), sl(NI);
    for (uint32_t n = 0; n < N; ++n) {
      const uint32_t third = kind[n] == PCB_INPUT ? node2input[n] : n_pid0[n];
      const uint32_t reg = region[n] == PCB_NONE ? 0x3fffffffu : region[n];
      sn[n] = make_uint4(estart[n], ecount[n], third, (uint32_t)kind[n] | (reg << 2));
      if (kind[n] == PCB_INPUT) {
        // a leaf has no edges: the two words carry its parameter offset and categories | variable << 16, so that
        // the sampler's walk needs no second record (0xffffffff: too large to pack, read s_leaf)
        const uint32_t i = node2input[n];
        const bool fits = in_poff[i] < 0xffffffffull && in_cats[i] < 65536u && in_var[i] < 65536u;
        sn[n].x = fits ? (uint32_t)in_poff[i] : 0xffffffffu;
        sn[n].y = fits ? (in_cats[i] | (in_var[i] << 16)) : 0u;
      }
    }
    for (uint32_t i = 0; i < NI; ++i)
      sl[i] = make_uint4((uint32_t)(in_poff[i] & 0xffffffffu), (uint32_t)(in_poff[i] >> 32), in_cats[i], in_var[i]);
    PCB_TRY(upload(&c->s_node, sn, &bytes));
    PCB_TRY(upload(&c->s_leaf, sl, &bytes));
  }
  PCB_TRY(upload(&c->e_prime, e_prime, &bytes));
  PCB_TRY(upload(&c->e_sub, e_sub, &bytes));
  PCB_TRY(upload(&c->in_node, in_node, &bytes));
  PCB_TRY(upload(&c->in_var, in_var, &bytes));
  {  // per variable the smallest category count of its leaves: what an observed value must stay below
    std::vector<uint32_t> var_cats(d->num_vars, 0xffffffffu);
    for (uint32_t i = 0; i < NI; ++i) var_cats[in_var[i]] = std::min(var_cats[in_var[i]], in_cats[i]);
    PCB_TRY(upload(&c->var_cats, var_cats, &bytes));
    PCB_CUDA(cudaMalloc((void**)&c->check_word, 4 * sizeof(int32_t)));
  }
  PCB_TRY(upload(&c->in_cats, in_cats, &bytes));
  PCB_TRY(upload(&c->in_poff, in_poff, &bytes));
  PCB_TRY(upload(&c->in_foff, in_foff, &bytes));
  PCB_TRY(upload(&c->node2input, node2input, &bytes));
  PCB_TRY(upload(&c->n_head, node_head, &bytes));
  PCB_TRY(upload(&c->head_roots, c->h_head_roots, &bytes));
  PCB_TRY(upload(&c->up_all, up_all, &bytes));
  PCB_TRY(upload(&c->up_same, up_same, &bytes));
  PCB_TRY(upload(&c->up_sparse, up_sparse, &bytes));
  PCB_TRY(upload(&c->down_all, down_all, &bytes));
  PCB_TRY(upload(&c->down_sparse, down_sparse, &bytes));
  PCB_TRY(upload(&c->in_off, in_off, &bytes));
  PCB_TRY(upload(&c->in_ent, in_ent, &bytes));
  PCB_TRY(upload(&c->dense, c->h_dense, &bytes));
  PCB_TRY(upload(&c->grp_node, grp_node, &bytes));
  {  // leaf chunks: inputs sorted by variable (stable), cut every PCB_LEAF_CHUNK leaves
    std::vector<uint32_t> order(NI), lvar, loff;
    for (uint32_t i = 0; i < NI; ++i) order[i] = i;
    std::stable_sort(order.begin(), order.end(), [&](uint32_t a, uint32_t b) { return in_var[a] < in_var[b]; });
    for (uint32_t i = 0; i < NI; ++i) {
      bool cut = i == 0 || in_var[order[i]] != in_var[order[i - 1]] || (i - loff.back()) >= PCB_LEAF_CHUNK;
      if (cut) { lvar.push_back(in_var[order[i]]); loff.push_back(i); }
    }
    loff.push_back(NI);
    c->n_lchunks = (uint32_t)lvar.size();
    PCB_TRY(upload(&c->lchunk_var, lvar, &bytes));
    PCB_TRY(upload(&c->lchunk_off, loff, &bytes));
    PCB_TRY(upload(&c->lchunk_inputs, order, &bytes));
    std::vector<uint32_t> gvar, goff;
    for (uint32_t i = 0; i < NI; ++i) {
      bool cut = i == 0 || in_var[order[i]] != in_var[order[i - 1]] || (i - goff.back()) >= PCB_LEAF_GROUP;
      if (cut) { gvar.push_back(in_var[order[i]]); goff.push_back(i); }
    }
    goff.push_back(NI);
    c->n_lgrps = (uint32_t)gvar.size();
    PCB_TRY(upload(&c->lgrp_var, gvar, &bytes));
    PCB_TRY(upload(&c->lgrp_off, goff, &bytes));
  }
  PCB_CUDA(cudaMalloc((void**)&c->status, sizeof(int)));
  PCB_CUDA(cudaMemset(c->status, 0, sizeof(int)));
  {  // dense blocks run on the tensor cores unless PCB_DENSE_IMPL=simt asks for the fp32 SIMT kernels
    cudaDeviceProp prop;
    PCB_CUDA(cudaGetDeviceProperties(&prop, c->device));
    const char* impl = getenv("PCB_DENSE_IMPL");
    const bool simt = impl && std::string(impl) == "simt";
    // sm_100 only: the fp32 SIMT kernels are the cross-check of the tensor-core path and run only on request
    if (prop.major != 10 && !simt && !c->h_dense.empty())
      return pcb_fail(PCB_ERR_INVALID, "dense sum blocks need an sm_100 device (tcgen05); this device is sm_" +
                                           std::to_string(prop.major) + std::to_string(prop.minor));
    c->use_tc = prop.major == 10 && !simt;
    auto flag = [](const char* name) { const char* e = getenv(name); return e && atoi(e) != 0; };
    c->graph_enabled = !flag("PCB_NO_GRAPH");
    c->pdl = !flag("PCB_NO_PDL");
    c->fwd_split = !flag("PCB_NO_FWD_SPLIT");
    c->bwd_split = !flag("PCB_NO_BWD_SPLIT");
    c->early_update = flag("PCB_EARLY_UPDATE");
    c->sample_walk_warp = flag("PCB_SAMPLE_WALK_WARP");
    c->sample_exact_keys = flag("PCB_SAMPLE_EXACT_KEYS");
    if (const char* e = getenv("PCB_LEAF_FLOW_IMPL")) c->leaf_flow_impl = !strcmp(e, "sorted") ? 2 : !strcmp(e, "atomic") ? 1 : 0;
    if (const char* e = getenv("PCB_CHECKED")) c->checked = atoi(e) != 0;
    if (const char* e = getenv("PCB_TC_KSPLIT")) { int v = atoi(e); c->tc_ksplit = (v == 1 || v == 2 || v == 4) ? v : 0; }
    if (const char* e = getenv("PCB_TC_NSPLIT")) { int v = atoi(e); c->tc_nsplit = (v == 1 || v == 2 || v == 4) ? v : 0; }
    if (const char* e = getenv("PCB_TC_A_STAGES")) { int v = atoi(e); c->tc_a_stages = (v == 2 || v == 4 || v == 8) ? v : 0; }
    if (const char* e = getenv("PCB_EDGE_IMPL")) c->edge_ld = !strcmp(e, "ld");
    if (c->use_tc) PCB_TRY(pcb_dense_tc_prepare(c, &bytes));
  }
  c->device_bytes = bytes;
  return PCB_OK;
}

}  // namespace

// Reads the device status word that bounded waits raise; non-zero means a kernel gave up waiting.
int32_t pcb_check_status(pcb_circuit* c) {
  int h = 0;
  PCB_CUDA(cudaMemcpy(&h, c->status, sizeof(int), cudaMemcpyDeviceToHost));
  if (h != 0) return pcb_fail(PCB_ERR_CUDA, "a dense-block kernel gave up a bounded wait (status " + std::to_string(h) + ")");
  return PCB_OK;
}

extern "C" int32_t pcb_circuit_status(pcb_circuit* c) {
  PCB_REQUIRE(c, "null argument");
  PCB_CUDA(cudaSetDevice(c->device));
  PCB_CUDA(cudaDeviceSynchronize());
  return pcb_check_status(c);
}

namespace {

void free_circuit(pcb_circuit* c) {
  void* ptrs[] = {c->theta, c->aggr, c->kind, c->n_estart, c->n_ecount, c->n_pid0, c->n_region, c->e_prime,
                  c->e_sub, c->in_node, c->in_var, c->in_cats, c->in_poff, c->in_foff, c->node2input,
                  c->up_all, c->up_sparse, c->down_all, c->down_sparse, c->in_off, c->in_ent, c->dense,
                  c->grp_node, c->lchunk_var, c->lchunk_off, c->lchunk_inputs, c->status, c->w_img, c->dense_img, c->w_img16, c->dense_img16,
                  c->lgrp_var, c->lgrp_off, c->s_node, c->s_leaf, c->n_head, c->head_roots, c->up_same, c->var_cats, c->check_word};
  for (void* p : ptrs) if (p) cudaFree(p);
  if (c->ev_g0) cudaEventDestroy(c->ev_g0);
  if (c->ev_g1) cudaEventDestroy(c->ev_g1);
  if (c->gstream) cudaStreamDestroy(c->gstream);
  if (c->ev_fork2) cudaEventDestroy(c->ev_fork2);
  if (c->ev_join2) cudaEventDestroy(c->ev_join2);
  for (cudaEvent_t ev : {c->ev_c0, c->ev_c1, c->ev_c2, c->ev_c3}) if (ev) cudaEventDestroy(ev);
  if (c->comm_stream) cudaStreamDestroy(c->comm_stream);
  if (c->side2) cudaStreamDestroy(c->side2);
  if (c->ev_fork) cudaEventDestroy(c->ev_fork);
  if (c->ev_join) cudaEventDestroy(c->ev_join);
  if (c->side) cudaStreamDestroy(c->side);
}

}  // namespace

extern "C" int32_t pcb_circuit_create(const pcb_circuit_desc* desc, int32_t device, pcb_circuit** out) {
  PCB_REQUIRE(desc && out, "null argument");
  int ndev = 0;
  PCB_CUDA(cudaGetDeviceCount(&ndev));
  PCB_REQUIRE(device >= 0 && device < ndev, "device index out of range");
  PCB_CUDA(cudaSetDevice(device));
  pcb_circuit* c = new pcb_circuit();
  c->device = device;
  int32_t st = compile(desc, c);
  if (st != PCB_OK) { free_circuit(c); delete c; return st; }
  *out = c;
  return PCB_OK;
}

extern "C" int32_t pcb_comm_destroy(pcb_circuit* c);

extern "C" int32_t pcb_circuit_destroy(pcb_circuit* c) {
  if (!c) return PCB_OK;
  cudaSetDevice(c->device);
  if (c->comm) pcb_comm_destroy(c);
  free_circuit(c);
  delete c;
  return PCB_OK;
}

extern "C" int32_t pcb_circuit_get_info(const pcb_circuit* c, pcb_circuit_info* info) {
  PCB_REQUIRE(c && info, "null argument");
  info->num_nodes = c->N; info->num_edges = c->E; info->num_sum_edges = c->n_inner; info->num_up_layers = c->L;
  info->num_inner_params = c->n_inner; info->num_input_params = c->n_input_params; info->num_param_groups = c->n_groups;
  info->num_dense_blocks = c->n_dense; info->num_sum_regions = c->n_regions; info->max_group_size = c->max_group;
  info->max_num_cats = c->max_cats; info->num_dense_edges = c->dense_edges; info->device_bytes = c->device_bytes;
  info->num_heads = c->n_heads; info->reserved = 0;
  return PCB_OK;
}

extern "C" int32_t pcb_get_head_roots(pcb_circuit* c, uint32_t* roots_host, uint64_t n) {
  PCB_REQUIRE(c && roots_host, "null argument");
  PCB_REQUIRE(n == c->n_heads, "the circuit has a different number of heads");
  for (uint32_t h = 0; h < c->n_heads; ++h) roots_host[h] = c->h_head_roots[h] + 1;
  return PCB_OK;
}

// ---- workspace ---------------------------------------------------------------------------------
extern "C" int32_t pcb_workspace_create(pcb_circuit* c, uint32_t max_batch, int32_t sets, pcb_workspace** out) {
  PCB_REQUIRE(c && out, "null argument");
  PCB_REQUIRE(max_batch >= 1, "max_batch must be positive");
  PCB_CUDA(cudaSetDevice(c->device));
  pcb_workspace* ws = new pcb_workspace();
  ws->c = c;
  ws->max_batch = max_batch;
  ws->ld = pcb_round_up(max_batch, 32);
  size_t n = (size_t)c->N * ws->ld * sizeof(float);
  cudaError_t e1 = cudaMalloc((void**)&ws->mars, n);
  cudaError_t e2 = e1 == cudaSuccess ? cudaMalloc((void**)&ws->flows, n) : e1;
  cudaError_t e3 = e2 == cudaSuccess ? cudaMalloc((void**)&ws->blk_mx, (size_t)std::max(1u, c->n_dense) * ws->ld * sizeof(float)) : e2;
  if (e3 != cudaSuccess) {
    if (ws->mars) cudaFree(ws->mars);
    if (ws->flows) cudaFree(ws->flows);
    delete ws;
    return pcb_fail(PCB_ERR_CUDA, std::string("workspace allocation: ") + cudaGetErrorString(e3));
  }
  if (cudaMalloc((void**)&ws->ids_stage, (size_t)max_batch * sizeof(int32_t)) != cudaSuccess) {
    pcb_workspace_destroy(ws);
    return pcb_fail(PCB_ERR_CUDA, "workspace allocation: row id staging");
  }
  {
    int32_t st = pcb_dense_edge_prepare_ws(ws);
    if (st != PCB_OK) { pcb_workspace_destroy(ws); return st; }
  }
  if (c->use_tc && c->n_dense) {
    // scratch of the K-split dense tiles: a launch that splits K stays within 296 CTAs, each with a
    // slot of at most 128 x 257 floats; one arrival counter per tile
    const size_t part_bytes = (size_t)296 * 128 * 257 * sizeof(float), ticket_bytes = 296 * sizeof(uint32_t);
    if (cudaMalloc((void**)&ws->mn_part, part_bytes) != cudaSuccess ||
        cudaMalloc((void**)&ws->mn_tickets, ticket_bytes) != cudaSuccess ||
        cudaMemset(ws->mn_tickets, 0, ticket_bytes) != cudaSuccess) {
      pcb_workspace_destroy(ws);
      return pcb_fail(PCB_ERR_CUDA, "workspace allocation: scratch of the K-split dense tiles");
    }
  }
  if (sets) {
    int32_t st = pcb_ws_ensure_sets(ws, max_batch, PCB_WS_NODES | PCB_WS_STACK | PCB_WS_EDGES);
    if (st != PCB_OK) { pcb_workspace_destroy(ws); return st; }
  }
  { std::lock_guard<std::mutex> g(c->ws_mu); c->workspaces.push_back(ws); }
  *out = ws;
  return PCB_OK;
}

int32_t pcb_ws_ensure_sets(pcb_workspace* ws, uint32_t S, int need) {
  pcb_circuit* c = ws->c;
  PCB_CUDA(cudaSetDevice(c->device));
  if ((need & (PCB_WS_NODES | PCB_WS_EDGES)) && S > ws->S_cap) {
    for (void* p : {(void*)ws->klds, (void*)ws->grads, (void*)ws->eprob, (void*)ws->cum}) if (p) cudaFree(p);
    ws->klds = ws->grads = ws->eprob = ws->cum = nullptr;
    ws->S_cap = S;
    // a handful of sets stays unpadded: the per-node values of neighbouring nodes then share 32-byte
    // sectors, which is what the gathers of a single-set KLD chain pay for
    ws->ldS = S <= 8 ? S : pcb_round_up(S, 32);
    ws->have_kld = false;
  }
  if ((need & PCB_WS_NODES) && !ws->klds) {
    PCB_CUDA(cudaMalloc((void**)&ws->klds, (size_t)c->N * ws->ldS * sizeof(float)));
    PCB_CUDA(cudaMalloc((void**)&ws->grads, (size_t)c->N * ws->ldS * sizeof(float)));
    ws->have_kld = false;
  }
  if ((need & PCB_WS_EDGES) && !ws->eprob) {   // the relaxed sampler's per-edge and per-group matrices
    PCB_CUDA(cudaMalloc((void**)&ws->eprob, (size_t)std::max(1u, c->n_inner) * ws->ldS * sizeof(float)));
    PCB_CUDA(cudaMalloc((void**)&ws->cum, (size_t)std::max(1u, c->n_groups) * ws->ldS * sizeof(float)));
  }
  // a pending entry of the walk stands for a sub-circuit over a scope disjoint from the other
  // pending ones, so V + 2 slots always suffice for a decomposable circuit
  ws->stack_cap = c->V + 2;
  if ((need & PCB_WS_STACK) && S > ws->stack_S) {
    if (ws->stack) cudaFree(ws->stack);
    ws->stack = nullptr;
    PCB_CUDA(cudaMalloc((void**)&ws->stack, (size_t)S * ws->stack_cap * sizeof(uint32_t)));
    ws->stack_S = S;
  }
  if (!ws->sample_status) PCB_CUDA(cudaMalloc((void**)&ws->sample_status, sizeof(int32_t)));
  return PCB_OK;
}

extern "C" int32_t pcb_workspace_destroy(pcb_workspace* ws) {
  if (!ws) return PCB_OK;
  cudaSetDevice(ws->c->device);
  {
    std::lock_guard<std::mutex> g(ws->c->ws_mu);
    auto& v = ws->c->workspaces;
    v.erase(std::remove(v.begin(), v.end(), ws), v.end());
  }
  if (ws->step_exec) cudaGraphExecDestroy(ws->step_exec);
  if (ws->kld_exec) cudaGraphExecDestroy(ws->kld_exec);
  for (void* p : {(void*)ws->mars, (void*)ws->flows, (void*)ws->blk_mx, (void*)ws->klds, (void*)ws->grads,
                  (void*)ws->eprob, (void*)ws->cum, (void*)ws->stack, (void*)ws->sample_status, (void*)ws->ids_stage, (void*)ws->ll_tmp, (void*)ws->mn_part, (void*)ws->mn_tickets,
                  (void*)ws->kld_t_dev})
    if (p) cudaFree(p);
  delete ws;
  return PCB_OK;
}

// ---- parameter accessors ---------------------------------------------------------------------
extern "C" int32_t pcb_get_params(pcb_circuit* c, float* params_host, uint64_t n) {
  PCB_REQUIRE(c && params_host, "null argument");
  PCB_REQUIRE(n == c->P, "parameter vector has the wrong length");
  PCB_CUDA(cudaSetDevice(c->device));
  PCB_CUDA(cudaDeviceSynchronize());
  PCB_TRY(pcb_check_status(c));
  PCB_CUDA(cudaMemcpy(params_host, c->theta, n * sizeof(float), cudaMemcpyDeviceToHost));
  return PCB_OK;
}
extern "C" int32_t pcb_set_params(pcb_circuit* c, const float* params_host, uint64_t n) {
  PCB_REQUIRE(c && params_host, "null argument");
  PCB_REQUIRE(n == c->P, "parameter vector has the wrong length");
  PCB_CUDA(cudaSetDevice(c->device));
  PCB_CUDA(cudaDeviceSynchronize());
  PCB_CUDA(cudaMemcpy(c->theta, params_host, n * sizeof(float), cudaMemcpyHostToDevice));
  c->w_img_valid = false;
  return PCB_OK;
}
extern "C" int32_t pcb_get_params_dev(pcb_circuit* c, float* params_dev, uint64_t n, pcb_stream s) {
  PCB_REQUIRE(c && params_dev, "null argument");
  PCB_REQUIRE(n == c->P, "parameter vector has the wrong length");
  PCB_CUDA(cudaSetDevice(c->device));
  PCB_CUDA(cudaMemcpyAsync(params_dev, c->theta, n * sizeof(float), cudaMemcpyDeviceToDevice, (cudaStream_t)s));
  return PCB_OK;
}
extern "C" int32_t pcb_set_params_dev(pcb_circuit* c, const float* params_dev, uint64_t n, pcb_stream s) {
  PCB_REQUIRE(c && params_dev, "null argument");
  PCB_REQUIRE(n == c->P, "parameter vector has the wrong length");
  PCB_CUDA(cudaSetDevice(c->device));
  PCB_CUDA(cudaMemcpyAsync(c->theta, params_dev, n * sizeof(float), cudaMemcpyDeviceToDevice, (cudaStream_t)s));
  c->w_img_valid = false;
  return PCB_OK;
}

// bpc.heap in the reference's layout: per leaf C log-probs, then C flow slots and the missing slot
extern "C" int32_t pcb_get_heap(pcb_circuit* c, float* heap_host, uint64_t n) {
  PCB_REQUIRE(c && heap_host, "null argument");
  PCB_REQUIRE(n == c->heap_len, "heap has the wrong length");
  PCB_CUDA(cudaSetDevice(c->device));
  PCB_CUDA(cudaDeviceSynchronize());
  std::vector<float> theta(c->theta_len ? c->theta_len : 1), aggr(c->aggr_len);
  PCB_CUDA(cudaMemcpy(theta.data(), c->theta, c->theta_len * sizeof(float), cudaMemcpyDeviceToHost));
  PCB_CUDA(cudaMemcpy(aggr.data(), c->aggr, c->aggr_len * sizeof(float), cudaMemcpyDeviceToHost));
  memset(heap_host, 0, n * sizeof(float));
  for (uint32_t i = 0; i < c->n_inputs; ++i) {
    uint32_t C = c->h_in_cats[i];
    float* h = heap_host + c->h_heap_start[i];
    memcpy(h, theta.data() + c->h_in_poff[i], C * sizeof(float));
    if (!c->h_in_fixed[i]) memcpy(h + C, aggr.data() + c->h_in_foff[i], (C + 1) * sizeof(float));
  }
  return PCB_OK;
}

// edge_aggr in down-edge order.  Only sum edges are aggregated: the reference's M-step
// (sgd/adam.jl:30-36, regularization/reg_em.jl:136-168) never reads the product-edge slots.
extern "C" int32_t pcb_get_edge_aggr(pcb_circuit* c, float* edge_aggr_host, uint64_t n) {
  PCB_REQUIRE(c && edge_aggr_host, "null argument");
  PCB_REQUIRE(n == c->E, "edge_aggr has the wrong length");
  PCB_CUDA(cudaSetDevice(c->device));
  PCB_CUDA(cudaDeviceSynchronize());
  PCB_TRY(pcb_check_status(c));
  std::vector<float> aggr(std::max<uint32_t>(1u, c->n_inner));
  PCB_CUDA(cudaMemcpy(aggr.data(), c->aggr, (size_t)c->n_inner * sizeof(float), cudaMemcpyDeviceToHost));
  for (uint32_t de = 0; de < c->E; ++de) {
    uint32_t p1 = c->h_edge2param[c->h_down2up[de]];
    edge_aggr_host[de] = p1 ? aggr[p1 - 1] : 0.0f;
  }
  return PCB_OK;
}

extern "C" int32_t pcb_get_edge2param(pcb_circuit* c, uint32_t* out, uint64_t n) {
  PCB_REQUIRE(c && out, "null argument");
  PCB_REQUIRE(n == c->E, "edge2param has the wrong length");
  memcpy(out, c->h_edge2param.data(), n * sizeof(uint32_t));
  return PCB_OK;
}
extern "C" int32_t pcb_get_sum_regions(pcb_circuit* c, uint32_t* out, uint64_t n) {
  PCB_REQUIRE(c && out, "null argument");
  PCB_REQUIRE(n == c->N, "node_region has the wrong length");
  memcpy(out, c->h_region1.data(), n * sizeof(uint32_t));
  return PCB_OK;
}

// ---- launch counters and per-class event timing ----------------------------------------------
static const char* kClassNames[PCB_K_COUNT] = {"leaf_forward", "sparse_up", "dense_fwd", "sparse_down",
                                               "dense_bwd_child", "dense_bwd_edge", "leaf_flow", "em_update",
                                               "misc", "allreduce", "dense_max", "w_image", "kld_adam", "sampling"};
extern "C" int32_t pcb_profile_num_classes(void) { return PCB_K_COUNT; }
extern "C" const char* pcb_profile_class_name(int32_t i) { return (i >= 0 && i < PCB_K_COUNT) ? kClassNames[i] : ""; }
extern "C" int32_t pcb_profile_enable(pcb_circuit* c, int32_t on) {
  PCB_REQUIRE(c, "null argument");
  c->prof.on = on != 0;
  return PCB_OK;
}
// Synchronises the device, adds up the event-bracketed time per kernel class (milliseconds) and
// returns the launch counters; reset != 0 clears both.
extern "C" int32_t pcb_profile_read(pcb_circuit* c, double* ms_out, uint64_t* launches_out, int32_t reset) {
  PCB_REQUIRE(c, "null argument");
  PCB_CUDA(cudaSetDevice(c->device));
  PCB_CUDA(cudaDeviceSynchronize());
  if (ms_out) {
    for (int i = 0; i < PCB_K_COUNT; ++i) ms_out[i] = 0.0;
    for (auto& e : c->prof.ev) {
      float ms = 0.0f;
      if (cudaEventElapsedTime(&ms, e.e0, e.e1) == cudaSuccess) ms_out[e.cls] += ms;
    }
  }
  if (launches_out) for (int i = 0; i < PCB_K_COUNT; ++i) launches_out[i] = c->prof.launches[i];
  if (reset) {
    for (auto& e : c->prof.ev) { cudaEventDestroy(e.e0); cudaEventDestroy(e.e1); }
    c->prof.ev.clear();
    for (int i = 0; i < PCB_K_COUNT; ++i) c->prof.launches[i] = 0;
  }
  return PCB_OK;
}
