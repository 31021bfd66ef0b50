"""Host-side mirror of the reference's call surface for the probabilistic-circuit hot path.

Same names and argument meaning as the Julia functions they stand for; every one of them
forwards to libpcb200.so through the C ABI of include/pcb200.h:

  CuMetaBitsProbCircuit(pc)             VariationalJuice.jl/src/bits_circuit.jl:5-113
  num_parameters / num_nodes / num_edges                         bits_circuit.jl:119-131
  vectorize_parameters / update_parameters                       src/misc.jl:5-135
  loglikelihoods(bpc, data; batch_size)                          regularization/reg_likelihood.jl:139-162
  mini_batch_em(bpc, data, epochs; batch_size, pseudocount, param_inertia, param_inertia_end,
                flow_memory, shuffle, weights)                   regularization/reg_em.jl:208-336
  full_batch_em                                                  (one step over all rows, inertia 0)
  mini_batch_em_with_reg / loglikelihoods_probcat                the same two under the names the experiment
                                                                 scripts call (reg_em.jl:208, reg_likelihood.jl:139)
  kld / kld_backward                                             queries/kld.jl:177-206, 593-649
  kld_preallocation / kld_with_prealloc / kld_backward_with_prealloc / kld_free_mem
                                                                 utils/cuda_preallocation.jl:6-78 (what PCVAE calls)
  gumbel_sample (soft) / sample (hard Gumbel-max)                queries/sample.jl:349-383
  gumbel_sample_preallocation / gumbel_sample_with_prealloc      utils/cuda_preallocation.jl:150-203

torch is used for device buffers and streams only.
"""
from __future__ import annotations

import ctypes as C
from typing import List, Optional, Sequence, Tuple, Union

import numpy as np
import torch

from . import _lib
from .circuit import FlatCircuit, PCNode, compile_circuit, compile_multihead

ArrayLike = Union[np.ndarray, torch.Tensor]


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None else C.c_void_p(t.data_ptr())


def _stream(device) -> C.c_void_p:
    return C.c_void_p(torch.cuda.current_stream(device).cuda_stream)


class DeviceData:
    """A data matrix [num_rows, num_vars] of uint8 categories resident on the GPU in the
    reference's column-major layout (stored as a contiguous [num_vars, num_rows] tensor)."""

    def __init__(self, data: ArrayLike, device, miss: Optional[ArrayLike] = None):
        self.t = self._put(data, device)
        self.miss = None if miss is None else self._put(miss, device)
        self.num_vars, self.num_rows = int(self.t.shape[0]), int(self.t.shape[1])

    @classmethod
    def from_colmajor(cls, t: torch.Tensor, miss: Optional[torch.Tensor] = None) -> "DeviceData":
        """Wrap a CUDA uint8 tensor that already is [num_vars, num_rows] contiguous."""
        assert t.is_cuda and t.dtype == torch.uint8 and t.is_contiguous() and t.dim() == 2
        self = cls.__new__(cls)
        self.t, self.miss = t, miss
        self.num_vars, self.num_rows = int(t.shape[0]), int(t.shape[1])
        return self

    @staticmethod
    def _put(a: ArrayLike, device) -> torch.Tensor:
        if isinstance(a, np.ndarray):
            a = torch.from_numpy(np.ascontiguousarray(a.T.astype(np.uint8, copy=False)))
        else:
            a = a.to(torch.uint8).t().contiguous()
        return a.to(device, non_blocking=True)


class CuMetaBitsProbCircuit:
    """Compiled circuit on one GPU (cu(BitsProbCircuit) + the flat parameter maps)."""

    def __init__(self, pc: Union[FlatCircuit, PCNode], device: int = 0):
        if not torch.cuda.is_available():
            raise _lib.PcbError(-1, "pcb200 needs a CUDA device; there is no CPU fallback")
        self.fc = pc if isinstance(pc, FlatCircuit) else compile_circuit(pc)
        self.device = torch.device("cuda", device)
        self.lib = _lib.lib()
        h = C.c_void_p()
        desc = self.fc.desc()
        _lib.check(self.lib.pcb_circuit_create(C.byref(desc), device, C.byref(h)))
        self.handle = h
        self.info = _lib.PcbCircuitInfo()
        _lib.check(self.lib.pcb_circuit_get_info(self.handle, C.byref(self.info)))
        self._ws = {}
        self.edge2param = np.zeros(self.fc.num_edges, np.uint32)
        _lib.check(self.lib.pcb_get_edge2param(self.handle, self.edge2param.ctypes.data, self.fc.num_edges))
        self.param2edge = (np.nonzero(self.edge2param)[0] + 1).astype(np.uint32)

    def __del__(self):
        try:
            for ws in self._ws.values():
                self.lib.pcb_workspace_destroy(ws)
            self.lib.pcb_circuit_destroy(self.handle)
        except Exception:
            pass

    def workspace(self, max_batch: int):
        """prep_memory: one workspace per maximal batch size, grown on demand."""
        for cap, ws in self._ws.items():
            if cap >= max_batch:
                return ws
        ws = C.c_void_p()
        _lib.check(self.lib.pcb_workspace_create(self.handle, max_batch, 0, C.byref(ws)))
        self._ws[max_batch] = ws
        return ws

    def free_workspaces(self):
        for ws in self._ws.values():
            self.lib.pcb_workspace_destroy(ws)
        self._ws = {}

    # ---- counters ----
    @property
    def num_inner_params(self) -> int:
        return int(self.info.num_inner_params)

    @property
    def num_input_params(self) -> int:
        return int(self.info.num_input_params)

    @property
    def num_param_groups(self) -> int:
        return int(self.info.num_param_groups)

    def sum_regions(self) -> np.ndarray:
        out = np.zeros(self.fc.num_nodes, np.uint32)
        _lib.check(self.lib.pcb_get_sum_regions(self.handle, out.ctypes.data, out.shape[0]))
        return out

    # ---- parity accessors ----
    def heap(self) -> np.ndarray:
        out = np.zeros(self.fc.heap.shape[0], np.float32)
        _lib.check(self.lib.pcb_get_heap(self.handle, out.ctypes.data, out.shape[0]))
        return out

    def edge_aggr(self) -> np.ndarray:
        out = np.zeros(self.fc.num_edges, np.float32)
        _lib.check(self.lib.pcb_get_edge_aggr(self.handle, out.ctypes.data, out.shape[0]))
        return out

    def _matrix(self, fn, ws, B) -> np.ndarray:
        out = np.zeros((B, self.fc.num_nodes), np.float32, order="F")
        _lib.check(fn(self.handle, ws, out.ctypes.data, out.size))
        return out

    def mars(self, ws, B) -> np.ndarray:
        return self._matrix(self.lib.pcb_get_mars, ws, B)

    def flows(self, ws, B) -> np.ndarray:
        return self._matrix(self.lib.pcb_get_flows, ws, B)

    # ---- launch accounting ----
    def profile_enable(self, on: bool) -> None:
        _lib.check(self.lib.pcb_profile_enable(self.handle, int(on)))

    def profile_read(self, reset: bool = True) -> dict:
        """{kernel class: (milliseconds under event timing, launches)} since the last reset."""
        n = self.lib.pcb_profile_num_classes()
        ms = (C.c_double * n)()
        cnt = (C.c_uint64 * n)()
        _lib.check(self.lib.pcb_profile_read(self.handle, C.cast(ms, C.c_void_p), C.cast(cnt, C.c_void_p), int(reset)))
        return {self.lib.pcb_profile_class_name(i).decode(): (float(ms[i]), int(cnt[i])) for i in range(n)}

    # ---- multi-GPU ----
    def attach_comm(self, unique_id: bytes, rank: int, nranks: int):
        buf = (C.c_uint8 * 128).from_buffer_copy(unique_id)
        _lib.check(self.lib.pcb_comm_init(self.handle, C.cast(buf, C.c_void_p), rank, nranks))


    def detach_comm(self):
        """Drop the communicator: later steps run on this GPU alone."""
        _lib.check(self.lib.pcb_comm_destroy(self.handle))

    def comm_poll(self):
        """Raise if NCCL reports an asynchronous error of the communicator."""
        _lib.check(self.lib.pcb_comm_poll(self.handle))

    def comm_wait(self, timeout_s: float, stream=None):
        """Bounded replacement for `torch.cuda.synchronize()` after steps with a collective: returns
        when the stream has drained; on an NCCL error or after `timeout_s` the communicator is
        aborted and a PcbError raised (then `detach_comm()` before the next step)."""
        st = torch.cuda.current_stream(self.device) if stream is None else stream
        _lib.check(self.lib.pcb_comm_wait(self.handle, C.c_void_p(st.cuda_stream), int(timeout_s * 1000)))

    def comm_abort(self):
        """End the communicator without waiting for its collectives."""
        _lib.check(self.lib.pcb_comm_abort(self.handle))


def comm_unique_id() -> bytes:
    buf = (C.c_uint8 * 128)()
    _lib.check(_lib.lib().pcb_comm_unique_id(C.cast(buf, C.c_void_p)))
    return bytes(buf)


def num_parameters(mbpc: CuMetaBitsProbCircuit) -> int:
    return mbpc.num_inner_params + mbpc.num_input_params


def num_nodes(mbpc: CuMetaBitsProbCircuit) -> int:
    return int(mbpc.info.num_nodes)


def num_edges(mbpc: CuMetaBitsProbCircuit) -> int:
    return int(mbpc.info.num_edges)


def vectorize_parameters(mbpc: CuMetaBitsProbCircuit, params: Optional[torch.Tensor] = None):
    """Copy the parameters from `mbpc` to `params` (a CUDA float vector) or return them as numpy."""
    n = num_parameters(mbpc)
    if params is not None:
        assert params.numel() == n and params.is_cuda and params.dtype == torch.float32
        _lib.check(mbpc.lib.pcb_get_params_dev(mbpc.handle, _ptr(params), n, _stream(mbpc.device)))
        return params
    out = np.zeros(n, np.float32)
    _lib.check(mbpc.lib.pcb_get_params(mbpc.handle, out.ctypes.data, n))
    return out


def update_parameters(mbpc: CuMetaBitsProbCircuit, params: ArrayLike) -> None:
    """Copy the parameters from `params` to `mbpc`."""
    n = num_parameters(mbpc)
    if isinstance(params, torch.Tensor) and params.is_cuda:
        assert params.numel() == n and params.dtype == torch.float32 and params.is_contiguous()
        _lib.check(mbpc.lib.pcb_set_params_dev(mbpc.handle, _ptr(params), n, _stream(mbpc.device)))
        return
    p = np.ascontiguousarray(np.asarray(params, dtype=np.float32).reshape(-1))
    assert p.shape[0] == n, f"{n} != {p.shape[0]}"
    _lib.check(mbpc.lib.pcb_set_params(mbpc.handle, p.ctypes.data, n))


def _as_data(mbpc, data) -> DeviceData:
    return data if isinstance(data, DeviceData) else DeviceData(data, mbpc.device)


def forward(mbpc, data, row_ids: Optional[torch.Tensor] = None, row_start: int = 1, B: Optional[int] = None,
            ll_out: Optional[torch.Tensor] = None):
    """eval_circuit on one batch; returns (workspace, B).  row_ids: 1-based int32 CUDA tensor."""
    data = _as_data(mbpc, data)
    if B is None:
        B = int(row_ids.numel()) if row_ids is not None else data.num_rows - (row_start - 1)
    ws = mbpc.workspace(B)
    _lib.check(mbpc.lib.pcb_forward(mbpc.handle, ws, _ptr(data.t), _ptr(data.miss), data.num_rows, _ptr(row_ids),
                                    row_start, B, _ptr(ll_out), _stream(mbpc.device)))
    return ws, B


def backward(mbpc, ws, weights: Optional[torch.Tensor] = None) -> None:
    _lib.check(mbpc.lib.pcb_backward(mbpc.handle, ws, _ptr(weights), _stream(mbpc.device)))


def loglikelihoods(mbpc: CuMetaBitsProbCircuit, data, batch_size: int = 512) -> torch.Tensor:
    """Per-row log-likelihoods, batches of consecutive rows (reg_likelihood.jl:139-162)."""
    data = _as_data(mbpc, data)
    out = torch.empty(data.num_rows, dtype=torch.float32, device=mbpc.device)
    for start in range(0, data.num_rows, batch_size):
        b = min(batch_size, data.num_rows - start)
        forward(mbpc, data, None, start + 1, b, out[start:start + b])
    return out


def em_step(mbpc, data, row_ids=None, row_start=1, B=None, pseudocount=0.1, inertia=0.0, clear_rate=0.0,
            weights=None, ll_sum: Optional[torch.Tensor] = None):
    """Per-batch body of mini_batch_em_with_reg (reg_em.jl:273-301)."""
    data = _as_data(mbpc, data)
    if B is None:
        B = int(row_ids.numel()) if row_ids is not None else data.num_rows - (row_start - 1)
    ws = mbpc.workspace(B)
    _lib.check(mbpc.lib.pcb_em_step(mbpc.handle, ws, _ptr(data.t), _ptr(data.miss), data.num_rows, _ptr(row_ids),
                                    row_start, B, _ptr(weights), clear_rate, pseudocount, inertia, _ptr(ll_sum),
                                    _stream(mbpc.device)))
    return ws


def _is_colmajor(t: torch.Tensor) -> bool:
    """First index fastest; the stride of an index of extent one is free."""
    want = 1
    for n, st in zip(t.shape, t.stride()):
        if n != 1 and st != want:
            return False
        want *= n
    return True


def _evidence(mbpc, data, soft, head_mask, row_ids, row_start, B, soft_reg, soft_reg_width):
    """Fill a pcb_evidence; returns (struct, B, keep-alive tuple)."""
    ev = _lib.PcbEvidence()
    keep = []
    if data is not None:
        data = _as_data(mbpc, data)
        ev.data_dev, ev.miss_dev, num_rows = _ptr(data.t), _ptr(data.miss), data.num_rows
        keep.append(data)
    if soft is not None:
        # [rows, V, C] with the rows fastest, as a Julia CuArray of that size lies in memory
        assert soft.is_cuda and soft.dtype == torch.float32 and soft.dim() == 3
        assert _is_colmajor(soft), "soft evidence must be column-major"
        ev.soft_dev, num_rows = _ptr(soft), soft.shape[0]
    if head_mask is not None:
        assert head_mask.is_cuda and head_mask.dtype == torch.float32 and head_mask.dim() == 2
        assert _is_colmajor(head_mask), "head mask must be column-major"
        assert head_mask.shape[0] == num_rows
        ev.head_mask_dev = _ptr(head_mask)
    if B is None:
        B = int(row_ids.numel()) if row_ids is not None else num_rows - (row_start - 1)
    ev.num_rows, ev.row_ids_dev, ev.row_start, ev.B = num_rows, _ptr(row_ids), row_start, B
    ev.soft_reg, ev.soft_reg_width = soft_reg, soft_reg_width
    keep += [soft, head_mask, row_ids]
    return ev, B, keep


def colmajor(a: ArrayLike, device) -> torch.Tensor:
    """A float32 CUDA tensor with the first index fastest (the layout of a Julia CuArray)."""
    t = torch.as_tensor(np.asarray(a, np.float32) if not torch.is_tensor(a) else a, dtype=torch.float32)
    perm = list(range(t.dim()))[::-1]
    return t.permute(*perm).contiguous().to(device).permute(*perm)


def forward_ex(mbpc, data=None, soft: Optional[torch.Tensor] = None, head_mask: Optional[torch.Tensor] = None,
               row_ids: Optional[torch.Tensor] = None, row_start: int = 1, B: Optional[int] = None,
               soft_reg: float = 0.0, soft_reg_width: int = 1, ll_out: Optional[torch.Tensor] = None):
    """eval_circuit on soft evidence (init_mar!_with_reg_cat, regularization/reg_likelihood.jl:51-91), with
    soft regularisation of the leaves (reg_likelihood.jl:4-49) and / or on a multi-head circuit
    (eval_multi_head_pc, src-jl/multi_head_pc/likelihood.jl:18-31); returns (workspace, B)."""
    ev, B, keep = _evidence(mbpc, data, soft, head_mask, row_ids, row_start, B, soft_reg, soft_reg_width)
    ws = mbpc.workspace(B)
    _lib.check(mbpc.lib.pcb_forward_ex(mbpc.handle, ws, C.byref(ev), _ptr(ll_out), _stream(mbpc.device)))
    return ws, B


def em_step_ex(mbpc, data=None, soft=None, head_mask=None, row_ids=None, row_start=1, B=None, pseudocount=0.1,
               inertia=0.0, clear_rate=0.0, weights=None, soft_reg=0.0, soft_reg_width=1,
               ll_sum: Optional[torch.Tensor] = None):
    """Per-batch body of mini_batch_em_with_reg (reg_em.jl:273-301) / mini_batch_em_for_multihead_pc
    (src-jl/multi_head_pc/em.jl:58-83) on the general forms of evidence."""
    ev, B, keep = _evidence(mbpc, data, soft, head_mask, row_ids, row_start, B, soft_reg, soft_reg_width)
    ws = mbpc.workspace(B)
    _lib.check(mbpc.lib.pcb_em_step_ex(mbpc.handle, ws, C.byref(ev), _ptr(weights), clear_rate, pseudocount, inertia,
                                       _ptr(ll_sum), _stream(mbpc.device)))
    return ws


def per_sample_normalized_flows(mbpc: CuMetaBitsProbCircuit, data, params: Optional[torch.Tensor] = None,
                                batch_size: int = 512) -> torch.Tensor:
    """`per_sample_normalized_flows(mbpc, data[, params]; batch_size)` (queries/flow.jl:417-494): a
    [rows, P] tensor (row index fastest, as the reference's CuMatrix) with, per data row, the log of every
    parameter's share of the flow of its sum node / leaf.  `params`: None for the circuit's own
    parameters, else [rows, P] log-parameters with the row index fastest, one vector per data row."""
    data = _as_data(mbpc, data)
    rows, P = data.num_rows, num_parameters(mbpc)
    if params is not None:
        assert params.is_cuda and params.dtype == torch.float32 and tuple(params.shape) == (rows, P)
        assert _is_colmajor(params), "per-row parameters must be column-major"
    out = torch.empty((P, rows), dtype=torch.float32, device=mbpc.device).t()   # [rows, P], rows fastest; every column is written
    ws = mbpc.workspace(min(batch_size, rows))
    for start in range(0, rows, batch_size):
        b = min(batch_size, rows - start)
        ev, _, keep = _evidence(mbpc, data, None, None, None, start + 1, b, 0.0, 1)
        _lib.check(mbpc.lib.pcb_normalized_flows(mbpc.handle, ws, C.byref(ev), _ptr(params), _ptr(out),
                                                 _stream(mbpc.device)))
    return out


def normalize_params(mbpc: CuMetaBitsProbCircuit, params: torch.Tensor, undo: bool = False) -> torch.Tensor:
    """`normalize_params(mbpc, params; undo)` (misc.jl:448-480) on a [S, P] CUDA tensor with the set index
    fastest, in place: leaves become probabilities, sum groups log-normalised."""
    assert params.is_cuda and params.dtype == torch.float32 and params.dim() == 2
    assert _is_colmajor(params) and params.shape[1] == num_parameters(mbpc)
    _lib.check(mbpc.lib.pcb_normalize_params(mbpc.handle, _ptr(params), params.shape[0], int(undo), _stream(mbpc.device)))
    return params


def map_pc_parameters(params1: torch.Tensor, params2: torch.Tensor, ids1: torch.Tensor, ids2: torch.Tensor) -> torch.Tensor:
    """The device half of `map_pc_parameters` (utils/map_params.jl:12-50): params1[:, ids1] = params2[:, ids2]
    with 1-based int32 / uint32 id vectors on the device (the caller computed the matching once)."""
    assert params1.is_cuda and params2.is_cuda and params1.shape[0] == params2.shape[0]
    assert _is_colmajor(params1) and _is_colmajor(params2)
    assert ids1.numel() == ids2.numel() and ids1.is_cuda and ids2.is_cuda and ids1.element_size() == 4 and ids2.element_size() == 4
    _lib.check(_lib.lib().pcb_map_param_columns(_ptr(params1), _ptr(params2), params1.shape[0], _ptr(ids1), _ptr(ids2),
                                                ids1.numel(), _stream(params1.device)))
    return params1


def normalized_flows(mbpc_xz: CuMetaBitsProbCircuit, mbpc_z: CuMetaBitsProbCircuit, data, mapping,
                     batch_size: int = 512) -> torch.Tensor:
    """`normalized_flows_with_prealloc(mbpc_xz, mbpc_z, data)` (utils/cuda_preallocation.jl:287-304): the
    normalised flows of the joint circuit, copied onto the latent circuit's parameters through
    `mapping` = (ids_z, ids_xz), clamped to [-20, 0] and normalised; returns [rows, P_z]."""
    nf = per_sample_normalized_flows(mbpc_xz, data, None, batch_size)
    rows = nf.shape[0]
    pz = torch.zeros((num_parameters(mbpc_z), rows), dtype=torch.float32, device=mbpc_z.device).t()
    map_pc_parameters(pz, nf, mapping[0], mapping[1])
    pz.clamp_(-20.0, 0.0)
    return normalize_params(mbpc_z, pz, undo=False)


def conditioned_td_prob(mbpc: CuMetaBitsProbCircuit, marked_var: torch.Tensor, marked_cat: torch.Tensor,
                        node_probs: torch.Tensor) -> torch.Tensor:
    """`conditioned_td_prob` / `cond_td_prob_with_prealloc` (queries/td_prob.jl:277-291,
    utils/cuda_preallocation.jl): marked_var / marked_cat are int32 CUDA vectors over the nodes (0 = not
    marked, else the 1-based latent variable and category of `mark_nodes`), node_probs [S, Z1, Z2] with
    the set index fastest; returns [S, num_vars, max_num_cats] with the set index fastest."""
    assert node_probs.is_cuda and node_probs.dtype == torch.float32 and node_probs.dim() == 3 and _is_colmajor(node_probs)
    assert marked_var.dtype == torch.int32 and marked_cat.dtype == torch.int32
    assert marked_var.numel() == mbpc.fc.num_nodes and marked_cat.numel() == mbpc.fc.num_nodes
    S, Z1 = int(node_probs.shape[0]), int(node_probs.shape[1])
    V, Cm = mbpc.fc.num_vars, int(mbpc.info.max_num_cats)
    out = torch.empty((Cm, V, S), dtype=torch.float32, device=mbpc.device).permute(2, 1, 0)
    ws = mbpc.workspace(1)
    _lib.check(mbpc.lib.pcb_cond_td_prob(mbpc.handle, ws, _ptr(marked_var), _ptr(marked_cat), _ptr(node_probs), S, Z1,
                                         _ptr(out), _stream(mbpc.device)))
    return out


def pairwise_mi(data, num_cats: int, pseudocount: float = 0.1, device: int = 0) -> torch.Tensor:
    """`pairwise_MI_chunked(data; num_cats, pseudocount)` (utils/information.jl:98-157): the [V, V] matrix of
    pairwise mutual information of the columns of `data` ([rows, V] uint8), computed on the tensor cores."""
    if not torch.cuda.is_available():
        raise _lib.PcbError(-1, "pcb200 needs a CUDA device; there is no CPU fallback")
    dev = torch.device("cuda", device)
    d = data if isinstance(data, DeviceData) else DeviceData(data, dev)
    V = d.num_vars
    out = torch.empty((V, V), dtype=torch.float32, device=dev)
    with torch.cuda.device(dev):
        _lib.check(_lib.lib().pcb_pairwise_mi(_ptr(d.t), d.num_rows, V, num_cats, pseudocount, _ptr(out), _stream(dev)))
    return out


def learn_chow_liu_tree(data, num_cats: int, pseudocount: float = 0.1, device: int = 0) -> np.ndarray:
    """The Chow-Liu tree of `data` as hclt() builds it (structures/hclts.jl:4-40, customizable_hclt.jl:106-126):
    pairwise MI on the GPU, maximum spanning tree and rooting at the tree's centre on the host; returns
    parent[v] (-1 at the root), the input of `structures.hclt_flat`."""
    from . import structures as st
    mi = pairwise_mi(data, num_cats, pseudocount, device).cpu().numpy().astype(np.float64)
    v = mi.shape[0]
    return st.root_tree_at_center(v, st.max_spanning_tree(mi))


class CuMultiHeadBitsProbCircuit(CuMetaBitsProbCircuit):
    """`CuMultiHeadBitsProbCircuit(pcs)` (src-jl/multi_head_pc/bit_circuit.jl:4-56): several heads over
    shared sub-circuits, held as one flat circuit under a fake root whose edges no top-down pass follows."""

    def __init__(self, pcs, device: int = 0):
        if isinstance(pcs, FlatCircuit):
            fc = pcs
        else:
            fc, _ = compile_multihead(list(pcs))
        super().__init__(fc, device)
        n = int(self.info.num_heads)
        roots = np.zeros(n, np.uint32)
        _lib.check(self.lib.pcb_get_head_roots(self.handle, roots.ctypes.data_as(C.c_void_p), n))
        self.root_ids = roots

    @property
    def bpc(self):
        return self


def multihead_loglikelihoods(mhbpc: CuMultiHeadBitsProbCircuit, data, head_mask: Optional[torch.Tensor],
                             batch_size: int = 512) -> torch.Tensor:
    """`loglikelihoods(mhbpc, data, head_mask; batch_size)` (src-jl/multi_head_pc/likelihood.jl:35-66) and
    multihead_loglikelihoods_probcat (src/multi_head_pc/multi_head_pc_likelihood.jl:37-63): [rows] with a
    mask, [rows, heads] without."""
    data = _as_data(mhbpc, data)
    H = len(mhbpc.root_ids)
    rows = data.num_rows
    out = torch.empty(rows if head_mask is not None else (H, rows), dtype=torch.float32, device=mhbpc.device)
    for start in range(0, rows, batch_size):
        b = min(batch_size, rows - start)
        if head_mask is not None:
            forward_ex(mhbpc, data, None, head_mask, None, start + 1, b, ll_out=out[start:start + b])
        else:
            tmp = torch.empty((H, b), dtype=torch.float32, device=mhbpc.device)
            forward_ex(mhbpc, data, None, None, None, start + 1, b, ll_out=tmp)
            out[:, start:start + b] = tmp
    return out if head_mask is not None else out.t()


def mini_batch_em_for_multihead_pc(mhbpc: CuMultiHeadBitsProbCircuit, data, head_mask: torch.Tensor, num_epochs: int,
                                   batch_size: int, pseudocount: float, soft_reg: float = 0.0, soft_reg_width: int = 1,
                                   param_inertia: float = 0.0, param_inertia_end: Optional[float] = None,
                                   flow_memory: float = 0.0, shuffle: str = "each_epoch", weights=None,
                                   seed: Optional[int] = None, verbose: bool = False) -> List[float]:
    """mini_batch_em_for_multihead_pc (src-jl/multi_head_pc/em.jl:1-100)."""
    return _mini_batch_loop(mhbpc, data, None, head_mask, num_epochs, batch_size, pseudocount, soft_reg, soft_reg_width,
                            param_inertia, param_inertia_end, flow_memory, shuffle, weights, seed, verbose)


def mini_batch_em_soft(mbpc: CuMetaBitsProbCircuit, soft: torch.Tensor, num_epochs: int, batch_size: int,
                       pseudocount: float, param_inertia: float = 0.0, param_inertia_end: Optional[float] = None,
                       flow_memory: float = 0.0, shuffle: str = "each_epoch", weights=None,
                       seed: Optional[int] = None, verbose: bool = False) -> List[float]:
    """mini_batch_em_with_reg on a 3-D array of per-category log-weights (reg_em.jl:196-318 with
    `data isa CuArray{Float32,3}`: init_mar!_with_reg_cat / input_flows_circuit_with_reg_cat)."""
    return _mini_batch_loop(mbpc, None, soft, None, num_epochs, batch_size, pseudocount, 0.0, 1, param_inertia,
                            param_inertia_end, flow_memory, shuffle, weights, seed, verbose)


def _mini_batch_loop(mbpc, data, soft, head_mask, num_epochs, batch_size, pseudocount, soft_reg, soft_reg_width,
                     param_inertia, param_inertia_end, flow_memory, shuffle, weights, seed, verbose) -> List[float]:
    if data is not None:
        data = _as_data(mbpc, data)
    rows = data.num_rows if data is not None else soft.shape[0]
    assert batch_size <= rows
    num_batches = rows // batch_size   # the last incomplete batch is dropped
    dev = mbpc.device
    gen = torch.Generator(device="cpu")
    if seed is not None:
        gen.manual_seed(seed)
    ids = torch.empty(rows, dtype=torch.int32, device=dev)

    def do_shuffle():
        ids.copy_((torch.randperm(rows, generator=gen) + 1).to(torch.int32), non_blocking=False)

    if shuffle == "once":
        do_shuffle()
    elif shuffle == "none":
        ids.copy_(torch.arange(1, rows + 1, dtype=torch.int32))
    if param_inertia_end is None:
        param_inertia_end = param_inertia
    d_inertia = (param_inertia_end - param_inertia) / num_epochs
    rate = 0.0 if flow_memory == 0 else max(0.0, 1.0 - (batch_size + pseudocount) / flow_memory)
    lls_epoch = torch.zeros(num_batches, dtype=torch.float32, device=dev)
    out: List[float] = []
    for epoch in range(num_epochs):
        if shuffle == "each_epoch":
            do_shuffle()
        for b in range(num_batches):
            if shuffle == "each_batch":
                do_shuffle()
            em_step_ex(mbpc, data, soft, head_mask, ids[b * batch_size:(b + 1) * batch_size], 1, batch_size, pseudocount,
                       param_inertia, rate, weights, soft_reg, soft_reg_width, lls_epoch[b:b + 1])
        out.append(float(lls_epoch.sum().item()) / batch_size / num_batches)
        _lib.check(mbpc.lib.pcb_circuit_status(mbpc.handle))
        param_inertia += d_inertia
        if verbose:
            print(f"Mini-batch EM epoch {epoch + 1}; train LL {out[-1]}")
    return out


def mini_batch_em(mbpc: CuMetaBitsProbCircuit, data, num_epochs: int, batch_size: int, pseudocount: float,
                  param_inertia: float, param_inertia_end: Optional[float] = None, flow_memory: float = 0.0,
                  shuffle: str = "each_epoch", weights: Optional[torch.Tensor] = None, seed: Optional[int] = None,
                  verbose: bool = False) -> List[float]:
    """mini_batch_em_with_reg with soft_reg = 0 (reg_em.jl:208-336): returns the per-epoch mean
    train log-likelihood.  The last incomplete batch of an epoch is dropped, as in the reference."""
    data = _as_data(mbpc, data)
    n = data.num_rows
    assert batch_size <= n
    if param_inertia_end is None:
        param_inertia_end = param_inertia
    num_batches = n // batch_size
    rng = np.random.default_rng(seed)
    delta = (param_inertia_end - param_inertia) / num_epochs
    ll_epoch = torch.zeros(num_batches, dtype=torch.float32, device=mbpc.device)
    perm_dev = torch.arange(1, n + 1, dtype=torch.int32, device=mbpc.device)

    def do_shuffle():
        perm_dev.copy_(torch.from_numpy((rng.permutation(n) + 1).astype(np.int32)), non_blocking=False)

    if shuffle == "once":
        do_shuffle()
    out = []
    rate = 0.0 if flow_memory == 0 else max(0.0, 1.0 - (batch_size + pseudocount) / flow_memory)
    for epoch in range(num_epochs):
        if shuffle == "each_epoch":
            do_shuffle()
        for b in range(num_batches):
            if shuffle == "each_batch":
                do_shuffle()
            ids = perm_dev[b * batch_size:(b + 1) * batch_size]
            em_step(mbpc, data, ids, 1, batch_size, pseudocount, param_inertia, rate, weights, ll_epoch[b:b + 1])
        ll = float(ll_epoch.sum().item()) / batch_size / num_batches
        _lib.check(mbpc.lib.pcb_circuit_status(mbpc.handle))   # the loop synchronises here anyway (reg_em.jl:303)
        out.append(ll)
        param_inertia += delta
        if verbose:
            print(f"Mini-batch EM epoch {epoch + 1}/{num_epochs}; train LL {ll}")
    return out


def mini_batch_em_with_reg(mbpc: CuMetaBitsProbCircuit, data, num_epochs: int, batch_size: int, pseudocount: float,
                           soft_reg: float = 0.0, soft_reg_width: int = 1, ent_reg: float = 0.0,
                           param_inertia: float = 0.0, param_inertia_end: Optional[float] = None, flow_memory: float = 0.0,
                           shuffle: str = "each_epoch", weights: Optional[torch.Tensor] = None, seed: Optional[int] = None,
                           verbose: bool = False, **ignored) -> List[float]:
    """The name and keyword set the experiment scripts use (reg_em.jl:208-213).  `soft_reg` must be 0
    (the plain leaf lookup, reg_likelihood.jl:4-14 with soft_reg = 0); `ent_reg` is accepted and
    ignored as in the reference, whose entropy step is commented out (reg_em.jl:294-296); the
    *_mem / mine / maxe / debug keywords tune the reference's own kernels and are ignored."""
    if soft_reg != 0.0:
        raise _lib.PcbError(1, "soft_reg > 0 (soft-regularised leaves) is not built")
    return mini_batch_em(mbpc, data, num_epochs, batch_size, pseudocount, param_inertia, param_inertia_end, flow_memory,
                         shuffle, weights, seed, verbose)


def loglikelihoods_probcat(mbpc: CuMetaBitsProbCircuit, data, batch_size: int = 512) -> torch.Tensor:
    """reg_likelihood.jl:139-162 for hard evidence (uint8 categories)."""
    return loglikelihoods(mbpc, data, batch_size)


def full_batch_em(mbpc: CuMetaBitsProbCircuit, data, num_epochs: int, batch_size: int, pseudocount: float) -> List[float]:
    """Accumulate flows over all rows (in batches), then one update with inertia 0."""
    data = _as_data(mbpc, data)
    out = []
    st = _stream(mbpc.device)
    for _ in range(num_epochs):
        _lib.check(mbpc.lib.pcb_clear_flows(mbpc.handle, 0.0, st))
        lls = torch.empty(data.num_rows, dtype=torch.float32, device=mbpc.device)
        for start in range(0, data.num_rows, batch_size):
            b = min(batch_size, data.num_rows - start)
            ws, _ = forward(mbpc, data, None, start + 1, b, lls[start:start + b])
            backward(mbpc, ws)
        _lib.check(mbpc.lib.pcb_em_update(mbpc.handle, pseudocount, 0.0, st))
        out.append(float(lls.double().mean().item()))
    return out


# ---- KLD ------------------------------------------------------------------------------------------
def _params_matrix(mbpc, p: ArrayLike) -> torch.Tensor:
    """[S, P] parameters as a CUDA tensor in column-major storage (a contiguous [P, S] tensor)."""
    if isinstance(p, np.ndarray):
        p = torch.from_numpy(np.atleast_2d(p).astype(np.float32, copy=False))
    if p.dim() == 1:
        p = p[None, :]
    return p.to(mbpc.device).t().contiguous()


def kld(mbpc: CuMetaBitsProbCircuit, params1: ArrayLike, params2: ArrayLike):
    """Returns (klds[S], reuse): `reuse` is what kld_backward needs.  The reference hands back the
    host copies (klds_mat, edge_klds_mat) for the same purpose (kld.jl:203-205); here the node
    values stay on the device and `kld_matrices(mbpc, reuse)` produces those two matrices on demand."""
    p1, p2 = _params_matrix(mbpc, params1), _params_matrix(mbpc, params2)
    S = int(p1.shape[1])
    ws = mbpc.workspace(1)
    out = torch.empty(S, dtype=torch.float32, device=mbpc.device)
    _lib.check(mbpc.lib.pcb_kld(mbpc.handle, ws, _ptr(p1), _ptr(p2), S, _ptr(out), _stream(mbpc.device)))
    return out, (ws, p1, p2, S)


def kld_matrices(mbpc, reuse) -> Tuple[np.ndarray, np.ndarray]:
    """klds [S, N] and edge_klds [S, E] of a kld() call, for parity checks."""
    ws, p1, p2, S = reuse
    klds = np.zeros((S, mbpc.fc.num_nodes), np.float32, order="F")
    _lib.check(mbpc.lib.pcb_get_klds(mbpc.handle, ws, S, klds.ctypes.data))
    ek = torch.zeros(mbpc.fc.num_edges, S, dtype=torch.float32, device=mbpc.device)
    _lib.check(mbpc.lib.pcb_kld_edge_klds(mbpc.handle, ws, _ptr(p1), _ptr(p2), S, _ptr(ek), _stream(mbpc.device)))
    return klds, ek.t().cpu().numpy()


def kld_backward(mbpc: CuMetaBitsProbCircuit, params1=None, params2=None, reuse=None):
    """Gradients of KLD(p1 || p2) w.r.t. the log-parameters of both arguments, [S, P] each."""
    assert reuse is not None, "call kld() first and pass its reuse tuple"
    ws, p1, p2, S = reuse
    P = num_parameters(mbpc)
    g1 = torch.zeros(P, S, dtype=torch.float32, device=mbpc.device)
    g2 = torch.zeros(P, S, dtype=torch.float32, device=mbpc.device)
    _lib.check(mbpc.lib.pcb_kld_backward(mbpc.handle, ws, _ptr(p1), _ptr(p2), S, _ptr(g1), _ptr(g2),
                                         _stream(mbpc.device)))
    return g1.t(), g2.t()


# The preallocated forms PCVAE calls through pyjulia (src/models/pc_vae.py:88-92,131,194): buffers are
# module-level state, as the reference keeps them in Julia globals (cuda_preallocation.jl:12-25).
_prealloc = {}


def kld_preallocation(mbpc: CuMetaBitsProbCircuit, num_examples: int) -> None:
    P = num_parameters(mbpc)
    dev = mbpc.device
    _prealloc["kld"] = dict(S=num_examples, p1=torch.empty(P, num_examples, device=dev), p2=torch.empty(P, num_examples, device=dev),
                            g1=torch.empty(P, num_examples, device=dev), g2=torch.empty(P, num_examples, device=dev),
                            out=torch.empty(num_examples, device=dev), ws=mbpc.workspace(1))


def kld_free_mem() -> None:
    _prealloc.pop("kld", None)


def kld_with_prealloc(mbpc: CuMetaBitsProbCircuit, params1: ArrayLike, params2: ArrayLike) -> np.ndarray:
    """klds[:, end] as a host vector (cuda_preallocation.jl:47-61); the parameters are copied into the
    preallocated device matrices and kept for kld_backward_with_prealloc."""
    b = _prealloc["kld"]
    for dst, src in ((b["p1"], params1), (b["p2"], params2)):
        src = torch.as_tensor(src, dtype=torch.float32)
        assert tuple(src.shape) == (b["S"], dst.shape[0]), "shape differs from kld_preallocation"
        dst.copy_(src.t(), non_blocking=True)
    _lib.check(mbpc.lib.pcb_kld(mbpc.handle, b["ws"], _ptr(b["p1"]), _ptr(b["p2"]), b["S"], _ptr(b["out"]),
                                _stream(mbpc.device)))
    return b["out"].cpu().numpy()


def kld_backward_with_prealloc(mbpc: CuMetaBitsProbCircuit) -> Tuple[np.ndarray, np.ndarray]:
    """(param_grads1, param_grads2) of the last kld_with_prealloc call as host matrices [S, P]
    (cuda_preallocation.jl:63-78)."""
    b = _prealloc["kld"]
    b["g1"].zero_(); b["g2"].zero_()
    _lib.check(mbpc.lib.pcb_kld_backward(mbpc.handle, b["ws"], _ptr(b["p1"]), _ptr(b["p2"]), b["S"], _ptr(b["g1"]),
                                         _ptr(b["g2"]), _stream(mbpc.device)))
    return b["g1"].t().cpu().numpy(), b["g2"].t().cpu().numpy()


class Adam:
    """Adam on a flat log-parameter vector followed by re-normalisation (sgd/adam.jl:63-127)."""

    def __init__(self, mbpc: CuMetaBitsProbCircuit, lr=1e-2, beta1=0.9, beta2=0.999, eps=1e-8):
        P = num_parameters(mbpc)
        self.mbpc, self.lr, self.beta1, self.beta2, self.eps = mbpc, lr, beta1, beta2, eps
        self.m = torch.zeros(P, dtype=torch.float32, device=mbpc.device)
        self.v = torch.zeros(P, dtype=torch.float32, device=mbpc.device)
        self.t = 0

    def step(self, theta: torch.Tensor, grad: torch.Tensor, sign: float = -1.0):
        self.t += 1
        grad = grad.contiguous().view(-1)
        _lib.check(self.mbpc.lib.pcb_adam_step(self.mbpc.handle, _ptr(theta), _ptr(grad), _ptr(self.m), _ptr(self.v),
                                               self.t, self.lr, self.beta1, self.beta2, self.eps, sign,
                                               _stream(self.mbpc.device)))


class KldAdam:
    """KLD(q || p) + gradient + Adam step on q + re-normalisation as one library call per step
    (pcb_kld_adam_step): the chain of small launches of a single parameter set is captured as a CUDA
    graph on the second step and replayed afterwards.  `theta_q` (a CUDA float vector) is updated
    in place; `step()` returns the KLD before the update as a one-element CUDA tensor."""

    def __init__(self, mbpc: CuMetaBitsProbCircuit, theta_q: torch.Tensor, theta_p: torch.Tensor, lr=1e-2, beta1=0.9,
                 beta2=0.999, eps=1e-8):
        P = num_parameters(mbpc)
        assert theta_q.is_cuda and theta_p.is_cuda and theta_q.numel() == P and theta_p.numel() == P
        self.mbpc, self.q, self.p = mbpc, theta_q, theta_p.contiguous()
        self.lr, self.beta1, self.beta2, self.eps = lr, beta1, beta2, eps
        self.m = torch.zeros(P, dtype=torch.float32, device=mbpc.device)
        self.v = torch.zeros(P, dtype=torch.float32, device=mbpc.device)
        self.kld = torch.zeros(1, dtype=torch.float32, device=mbpc.device)
        self.ws = mbpc.workspace(1)
        self.t = 0

    def step(self) -> torch.Tensor:
        self.t += 1
        _lib.check(self.mbpc.lib.pcb_kld_adam_step(self.mbpc.handle, self.ws, _ptr(self.q), _ptr(self.p), _ptr(self.m),
                                                   _ptr(self.v), self.t, self.lr, self.beta1, self.beta2, self.eps,
                                                   _ptr(self.kld), _stream(self.mbpc.device)))
        return self.kld


# ---- sampling ---------------------------------------------------------------------------------------
def noise_shapes(mbpc: CuMetaBitsProbCircuit, S: int):
    """Shapes of the uniform buffers `sample` expects: u_sum [S, R, kmax], u_leaf [S, V, cmax]."""
    return ((S, int(mbpc.info.num_sum_regions), int(mbpc.info.max_group_size)),
            (S, mbpc.fc.num_vars, int(mbpc.info.max_num_cats)))


def sample(mbpc: CuMetaBitsProbCircuit, params: ArrayLike, u_sum: ArrayLike, u_leaf: ArrayLike) -> torch.Tensor:
    """Hard Gumbel-max samples x [S, V] (int32, 0-based categories) from caller-supplied uniforms."""
    p = _params_matrix(mbpc, params)
    us = torch.as_tensor(u_sum, dtype=torch.float32).to(mbpc.device).contiguous()
    ul = torch.as_tensor(u_leaf, dtype=torch.float32).to(mbpc.device).contiguous()
    S = int(ul.shape[0])
    shp = noise_shapes(mbpc, S)
    assert tuple(us.shape) == shp[0] and tuple(ul.shape) == shp[1], (us.shape, ul.shape, shp)
    ws = mbpc.workspace(1)
    x = torch.empty(mbpc.fc.num_vars, S, dtype=torch.int32, device=mbpc.device)
    _lib.check(mbpc.lib.pcb_sample_hard(mbpc.handle, ws, _ptr(p), int(p.shape[1]), _ptr(us), _ptr(ul), S, _ptr(x),
                                        _stream(mbpc.device)))
    return x.t()


def sample_static(mbpc: CuMetaBitsProbCircuit, params: torch.Tensor, u_sum: torch.Tensor, u_leaf: torch.Tensor,
                  x_out: torch.Tensor) -> torch.Tensor:
    """`sample` for callers whose memory pool must stay in charge: every buffer, the output
    included, is passed in as a CUDA tensor in the layout the C ABI takes (params [P, Sp]
    contiguous, x_out [V, S] int32) and the library allocates nothing (pcb_sample_hard_static)."""
    S = int(u_leaf.shape[0])
    _lib.check(mbpc.lib.pcb_sample_hard_static(mbpc.handle, _ptr(params), int(params.shape[1]), _ptr(u_sum),
                                               _ptr(u_leaf), S, _ptr(x_out), _stream(mbpc.device)))
    return x_out.t()


def gumbel_sample_preallocation(mbpc: CuMetaBitsProbCircuit, num_examples: int, num_vars: int, par_buffer_size: int) -> None:
    """cuda_preallocation.jl:150-187: the sampler's buffers live in the workspace here; this records
    the shapes the later calls are checked against."""
    assert num_vars == mbpc.fc.num_vars and par_buffer_size == int(mbpc.info.max_num_cats)
    _prealloc["sample"] = dict(S=num_examples, V=num_vars, C=par_buffer_size)


def gumbel_sample_with_prealloc(mbpc: CuMetaBitsProbCircuit, params: ArrayLike, temperature: float, no_gumbel: bool = False,
                                u: Optional[ArrayLike] = None) -> np.ndarray:
    """input_aggr_params as a host array [S, num_vars, par_buffer_size] (cuda_preallocation.jl:189-203)."""
    b = _prealloc["sample"]
    out = gumbel_sample(mbpc, params, b["V"], b["C"], temperature, no_gumbel=no_gumbel, u=u, S=b["S"])
    return out.cpu().numpy()


def gumbel_sample(mbpc: CuMetaBitsProbCircuit, params: ArrayLike, num_vars: int, par_buffer_size: int,
                  temperature: float, no_gumbel: bool = False, u: Optional[ArrayLike] = None, S: Optional[int] = None):
    """Relaxed top-down sampling: returns input_aggr_params [S, num_vars, par_buffer_size].
    The reference draws its noise in-kernel; here `u` ([S, num_inner_params] uniforms) is passed
    in, or no_gumbel=True selects the noise-free variant."""
    p = _params_matrix(mbpc, params)
    Sp = int(p.shape[1])
    S = S or Sp
    assert num_vars == mbpc.fc.num_vars and par_buffer_size == int(mbpc.info.max_num_cats)
    ud = None
    if not no_gumbel:
        assert u is not None, "pass uniforms `u` or no_gumbel=True"
        ud = torch.as_tensor(u, dtype=torch.float32).to(mbpc.device).t().contiguous()
    ws = mbpc.workspace(1)
    out = torch.empty(par_buffer_size, num_vars, S, dtype=torch.float32, device=mbpc.device)
    _lib.check(mbpc.lib.pcb_sample_soft(mbpc.handle, ws, _ptr(p), Sp, _ptr(ud), temperature, S, _ptr(out),
                                        _stream(mbpc.device)))
    return out.permute(2, 1, 0)
