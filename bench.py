#!/usr/bin/env python
"""Benchmark of the probabilistic-circuit hot path: forward + backward + EM update
(mini-batch EM step) on a seeded synthetic HCLT workload.

    python bench.py --gpus N --steps K --warmup W [--config cfg5|cfg2|...] [--impl reference]

One JSON line on rank 0.  `value` = samples/s of the whole job with data resident in HBM;
`e2e` = the same through the public API with host (pinned) batches copied in every step and the
batch log-likelihood read back; `roofline` = the dominant kernel class against the measured peak;
`cpu_baseline` = the CPU oracle (a restatement of the reference's algorithm) on a bounded sample.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

CONFIGS = {
    # name: (num_vars, latents k, global batch, data rows, description)
    "cfg5": dict(num_vars=3072, k=256, batch=2048, rows=50000, cats=256,
                 desc="HCLT 3072 vars x 256 cats, 256 latents (config 5), mini-batch EM B=2048"),
    "cfg2": dict(num_vars=3072, k=32, batch=512, rows=50000, cats=256,
                 desc="HCLT 3072 vars x 256 cats, 32 latents (config 2), mini-batch EM B=512"),
    "cfg5s": dict(num_vars=384, k=256, batch=2048, rows=8192, cats=256,
                  desc="reduced config 5: first 384 variables, 256 latents, B=2048 (profiling size)"),
    "tiny": dict(num_vars=48, k=32, batch=256, rows=2048, cats=256,
                 desc="tiny smoke workload: 48 variables, 32 latents, B=256"),
}
PSEUDOCOUNT, INERTIA = 0.1, 0.9  # step size 0.1


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return {"hbm_gbs": d["hbm_gbs"], "tflops": d.get("bf16_tflops_sustained", d["bf16_tflops"]), "which": "measured"}
    return {"hbm_gbs": 6650.0, "tflops": 1400.0, "which": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs.

    nvidia-smi needs a few hundred milliseconds to come up (longer on a box with eight GPUs), during which it
    queries every GPU of the machine: `start()` therefore launches it ahead of the warm-up steps and waits (at
    most three seconds) for its first line, `begin()` / `end()` bracket the timed region, and `summary()` uses
    the lines that arrived in between.  Used as a context manager it does all of that around the block.  One
    sampler per job is enough: ranks other than 0 pass enabled=False and run nothing."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int, enabled: bool = True, period_ms: int = 100):
        self.index, self.enabled, self.period_ms = index, enabled, period_ms
        self.rows, self.proc, self.t_begin, self.t_end = [], None, None, None

    def start(self, wait_s: float = 3.0):
        if not self.enabled or self.proc:
            return self
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.Q,
                                          "--format=csv,noheader,nounits", "-lms", str(self.period_ms)],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
            deadline = time.perf_counter() + wait_s
            while not self.rows and time.perf_counter() < deadline and self.proc.poll() is None:
                time.sleep(0.01)
        except Exception:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append((time.perf_counter(), [x.strip() for x in line.split(",")]))

    def begin(self):
        self.t_begin = time.perf_counter()

    def end(self):
        self.t_end = time.perf_counter()
        if self.proc:
            time.sleep(1.5e-3 * self.period_ms)   # one more line, taken while the last kernels still ran or just after
            self.proc.terminate()
            try:
                self.proc.wait(timeout=2)
            except Exception:
                self.proc.kill()

    def __enter__(self):
        self.start()
        self.begin()
        return self

    def __exit__(self, *a):
        self.end()

    def summary(self):
        lo = (self.t_begin or 0.0)
        hi = (self.t_end or float("inf")) + 2e-3 * self.period_ms
        rows = [r for t, r in self.rows if lo <= t <= hi]
        sm = [float(r[0]) for r in rows if len(r) >= 6 and r[0].replace(".", "").isdigit()]
        mx = [float(r[1]) for r in rows if len(r) >= 6 and r[1].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(len(r) >= 6 and r[2 + i].lower().startswith("active") for r in rows)]
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(sm)}


def build_workload(cfg, device, seed=3):
    from lvd_pg_b200 import synth
    images, fc = synth.image_hclt(cfg["k"], cfg["rows"], 32, 2.0, seed, device,
                                  num_vars=None if cfg["num_vars"] == 3072 else cfg["num_vars"])
    return images, fc


def algorithmic_work(fc, info, B):
    """Per-step algorithmic flops of the dense blocks and bytes of every kernel class, from the
    circuit's own counts (B examples; fp32 = 4 bytes)."""
    n_in = len(fc.input_node_ids)
    N = fc.num_nodes
    Ed = int(info.num_dense_edges)
    Es = int(info.num_inner_params)
    k = fc.meta.get("k", 1)
    dense_nodes = Ed // max(k, 1)           # parents in dense blocks
    work = {
        # three contractions of 2*B*k*k per block: values, child flows, edge statistics
        "dense_fwd": {"flops": 2.0 * B * Ed, "bytes": 4.0 * (B * dense_nodes * 3 + Ed)},
        "dense_bwd_child": {"flops": 2.0 * B * Ed, "bytes": 4.0 * (B * dense_nodes * 6 + Ed)},
        "dense_bwd_edge": {"flops": 2.0 * B * Ed, "bytes": 4.0 * (B * dense_nodes * 4 + 3 * Ed)},
        # leaf values written / leaf flows read once; the parameter tables and the data bytes are small
        # beside them; the leaf statistics are read-modify-written once per step
        "leaf_forward": {"bytes": 4.0 * B * n_in + B * fc.num_vars},
        "leaf_flow": {"bytes": 4.0 * B * n_in + B * fc.num_vars + 8.0 * (fc.num_input_params + n_in)},
        "sparse_up": {"bytes": 4.0 * B * (N - n_in - dense_nodes) * 3},
        "sparse_down": {"bytes": 4.0 * B * (N - 2 * dense_nodes) * 4},
        "em_update": {"bytes": 16.0 * (Es + fc.num_input_params)},
        "w_image": {"bytes": 20.0 * Ed},
    }
    return work


# DRAM bytes per dense block (256 parents x 256 children) at 2048 examples, dram__bytes_read.sum +
# dram__bytes_write.sum of one ncu capture of the largest launches of the 384-variable cut of the
# workload (profiles/dense_mn_kernels_cfg5s.md, profiles/dense_edge_tma_kernel_cfg5s.md); traffic grows in
# proportion to blocks x examples.
NCU_DRAM_BYTES_PER_BLOCK = {"dense_bwd_edge": 2445.3e6 / 287, "dense_bwd_child": 673.7e6 / 55, "dense_fwd": 407.1e6 / 55}


def measured_traffic(kernel_class, info, B, launches_per_step):
    """Per-launch DRAM traffic of a dense class scaled from the ncu capture, or None."""
    per_block = NCU_DRAM_BYTES_PER_BLOCK.get(kernel_class)
    if per_block is None or int(info.num_dense_blocks) == 0 or not launches_per_step:
        return None
    k2 = float(info.num_dense_edges) / float(info.num_dense_blocks)   # edges per block
    return per_block * (k2 / 65536.0) * (B / 2048.0) * int(info.num_dense_blocks) / launches_per_step


def host_threads():
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except Exception:
        return max(1, os.cpu_count() or 1)


def cpu_model():
    try:
        for line in open("/proc/cpuinfo"):
            if line.startswith("model name"):
                return line.split(":", 1)[1].strip()
    except Exception:
        pass
    return "unknown"


class CpuOracle:
    """The CPU arm: the oracle (a C restatement of the reference's per-(example, edge) algorithm),
    built -march=native on this machine, on every host thread the process may use (torchrun exports
    OMP_NUM_THREADS=1, so the count is set explicitly).  One EM step = E-step on `rows` rows (forward,
    backward, leaf statistics: linear in the rows) + the M-step over all parameters (independent of the
    rows).  Throughput is stated for the workload's full batch: B / (t_E * B / rows + t_M)."""

    def __init__(self, fc, images_cpu):
        from oracle import oracle as orc
        orc.use_native_build()
        self.orc, self.threads = orc, host_threads()
        orc.set_num_threads(self.threads)
        self.ref = fc.copy()
        self.images = images_cpu
        self.aggr = np.zeros(fc.num_edges, np.float32)

    def step(self, rows, first_row=0):
        orc, ref = self.orc, self.ref
        rows = max(1, min(rows, self.images.shape[0] - first_row))
        orc.set_row_block(max(1, min(16, rows // self.threads)))
        data = np.asfortranarray(self.images[first_row:first_row + rows])
        t0 = time.perf_counter()
        orc.clear_flows(ref, self.aggr, 0.0)
        mars = orc.forward(ref, data)
        flows, _ = orc.backward(ref, mars, self.aggr)
        orc.input_flows(ref, flows, data)
        t1 = time.perf_counter()
        orc.em_update(ref, self.aggr, PSEUDOCOUNT, INERTIA)
        t2 = time.perf_counter()
        return rows, t1 - t0, t2 - t1

    @staticmethod
    def full_batch_rate(B, rows, t_e, t_m):
        return B / (t_e * B / rows + t_m)

    def describe(self, B, rows, t_e, t_m):
        return {"value": self.full_batch_rate(B, rows, t_e, t_m), "unit": "samples/s", "cores": self.threads, "kind": "port",
                "sample": (f"E-step (forward, backward, leaf statistics) timed on {rows} rows of the same workload "
                           f"(full circuit) and scaled linearly to the batch of {B}; M-step timed in full"),
                "rows": rows, "threads": self.threads, "nproc": os.cpu_count(), "cpu_model": cpu_model(),
                "e_step_s": round(t_e, 3), "m_step_s": round(t_m, 3), "batch": B,
                "e_step_s_at_batch": round(t_e * B / rows, 2), "build": "gcc -O3 -march=native -fopenmp, fp32, no fast-math",
                "measured_samples_per_s_on_sample": rows / (t_e + t_m)}


def measure_cfg4(args, cpu_leg=True):
    """Config 4 (variational path): exact KLD(q || p) + gradient + Adam step, then hard sampling, on
    two HCLTs over 784 binary variables with 64 latents.  One GPU (a single parameter set has no
    batch dimension to shard).  Returns the JSON line as a dict."""
    import torch
    from lvd_pg_b200 import api, synth
    assert torch.cuda.is_available(), "bench.py needs a CUDA device (no CPU fallback)"
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    q, pcirc = synth.config4()
    m = api.CuMetaBitsProbCircuit(q, dev.index)
    theta_q = torch.from_numpy(np.asarray(api.vectorize_parameters(m), np.float32)).to(dev)
    mp = api.CuMetaBitsProbCircuit(pcirc, dev.index)
    theta_p = torch.from_numpy(np.asarray(api.vectorize_parameters(mp), np.float32)).to(dev)
    del mp
    P = int(theta_q.numel())
    opt = api.KldAdam(m, theta_q, theta_p, lr=1e-2, beta1=0.9, beta2=0.999, eps=1e-8)   # one library call per step
    klv = []

    def step():
        opt.step()   # the KLD of the step stays in opt.kld (device); nothing else is launched

    opt.step()
    klv.append(opt.kld.clone())
    for _ in range(max(args.warmup - 1, 2)):
        step()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(dev.index) as clocks:
        e0.record()
        for _ in range(args.steps):
            step()
        e1.record()
        torch.cuda.synchronize()
    us = e0.elapsed_time(e1) * 1e3 / args.steps
    klv.append(opt.kld.clone())
    # hard sampling of 4096 samples from q with caller-supplied uniforms (seed 5)
    S = 4096
    shp_s, shp_l = api.noise_shapes(m, S)
    g = torch.Generator(device=dev).manual_seed(5)
    u_sum = torch.rand(shp_s, generator=g, device=dev, dtype=torch.float32)
    u_leaf = torch.rand(shp_l, generator=g, device=dev, dtype=torch.float32)
    for _ in range(3):
        x = api.sample(m, theta_q, u_sum, u_leaf)
    torch.cuda.synchronize()
    reps = max(3, args.steps)
    e0.record()
    for _ in range(reps):
        x = api.sample(m, theta_q, u_sum, u_leaf)
    e1.record()
    torch.cuda.synchronize()
    samp_ms = e0.elapsed_time(e1) / reps
    # per-sample normalised flows of 512 rows with the circuit's own parameters (the encoder side of the
    # variational loop, utils/cuda_preallocation.jl:287-304): output [512, P]
    rows_nf = 512
    rng_nf = np.random.default_rng(9)
    data_nf = api.DeviceData(rng_nf.integers(0, 2, size=(rows_nf, q.num_vars)).astype(np.uint8), dev)
    api.update_parameters(m, theta_q)
    for _ in range(2):
        nf = api.per_sample_normalized_flows(m, data_nf, batch_size=rows_nf)
    torch.cuda.synchronize()
    e0.record()
    for _ in range(5):
        nf = api.per_sample_normalized_flows(m, data_nf, batch_size=rows_nf)
    e1.record()
    torch.cuda.synchronize()
    nf_ms = e0.elapsed_time(e1) / 5
    nf_bytes = 4.0 * rows_nf * P
    del nf
    peaks = measured_peaks()
    kld_bytes = 48.0 * P
    samp_bytes = 8.0 * S * (shp_s[1] * shp_s[2] + shp_l[1] * shp_l[2])
    cpu = None
    if cpu_leg and not args.no_cpu_baseline:
        from oracle import oracle as orc
        orc.lib()
        tq, tp = theta_q.cpu().numpy().copy(), theta_p.cpu().numpy()
        mm, vv = np.zeros_like(tq), np.zeros_like(tq)
        t0 = time.perf_counter()
        klds, ek = orc.kld(q, tq, tp)
        gr = orc.kld_backward(q, tq, tp, klds, ek)
        orc.adam_step(q, tq, gr["param_grads1"][0], mm, vv, 1)
        cdt = time.perf_counter() - t0
        cpu = {"value": cdt * 1e6, "unit": "us/step", "cores": orc.num_threads(), "kind": "port",
               "sample": "one KLD + gradient + Adam step of the same circuit pair"}
    line = {"metric": "us per KLD+grad+Adam step", "value": us, "unit": "us/step", "n_gpus": 1, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": us / 1e3, "higher_is_better": False, "scaling": "replicas only",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": "config 4: KLD(q||p) + grad + Adam, HCLT 784 binary vars, 64 latents; then hard sampling S=4096",
                       "params": P, "nodes": q.num_nodes, "edges": q.num_edges, "up_layers": int(m.info.num_up_layers)},
            "kld_last": float(klv[-1][0].item()), "kld_first": float(klv[0][0].item()),
            "roofline": {"bound": "hbm", "achieved": kld_bytes / (us * 1e-6) / 1e9, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                         "frac": kld_bytes / (us * 1e-6) / 1e9 / peaks["hbm_gbs"], "traffic": None,
                         "note": "latency-bound: one launch per layer on a single parameter set"},
            "sampling": {"samples_per_s": S / (samp_ms * 1e-3), "ms_per_call": samp_ms, "S": S,
                         "hbm_gbs": samp_bytes / (samp_ms * 1e-3) / 1e9, "hbm_frac": samp_bytes / (samp_ms * 1e-3) / 1e9 / peaks["hbm_gbs"]},
            "normalized_flows": {"rows": rows_nf, "ms_per_call": nf_ms, "rows_per_s": rows_nf / (nf_ms * 1e-3),
                                 "output_gbs": nf_bytes / (nf_ms * 1e-3) / 1e9,
                                 "note": "forward + backward + normalising kernels; the output is [rows, P] floats"},
            "clocks": clocks.summary(), "gpu_launches": int(sum(v[1] for v in m.profile_read(reset=True).values()))}
    if cpu:
        line["cpu_baseline"] = cpu
    return line


def measure_cfg2_step(steps=10, warmup=3):
    """Config 2 (3072 variables x 256 categories, 32 latents, B = 512): milliseconds per mini-batch EM
    step with the data resident on the GPU."""
    import torch
    from lvd_pg_b200 import api
    cfg = CONFIGS["cfg2"]
    dev = torch.device("cuda", torch.cuda.current_device())
    images, fc = build_workload(cfg, dev)
    m = api.CuMetaBitsProbCircuit(fc, dev.index)
    data = api.DeviceData(images, dev)
    rng = np.random.default_rng(321)
    ids = [torch.from_numpy((rng.permutation(data.num_rows)[:cfg["batch"]] + 1).astype(np.int32)).to(dev) for _ in range(steps + warmup)]
    ll = torch.zeros(1, device=dev)
    for i in range(warmup):
        api.em_step(m, data, ids[i], 1, cfg["batch"], PSEUDOCOUNT, INERTIA, 0.0, None, ll)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(warmup, warmup + steps):
        api.em_step(m, data, ids[i], 1, cfg["batch"], PSEUDOCOUNT, INERTIA, 0.0, None, ll)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / steps
    return {"workload": cfg["desc"], "ms_per_step": ms, "samples_per_s": cfg["batch"] / (ms * 1e-3), "steps": steps,
            "sum_edges": int(m.info.num_inner_params), "train_ll_last_batch": float(ll.item()) / cfg["batch"]}


def run_cfg3(args):
    """Config 3 (patch model): forward + backward + EM on 64 independent HCLTs (192 variables,
    128 latents, 256 categories), batch 256 images per circuit, all circuits of a step in flight
    together on their own streams.  With N GPUs the circuits are dealt out 64 / N per rank, no
    collective.  Prints its own JSON line."""
    import torch
    import torch.distributed as dist
    from lvd_pg_b200 import api, synth
    assert torch.cuda.is_available(), "bench.py needs a CUDA device (no CPU fallback)"
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    B = 256
    parts = synth.config3(device=dev)
    mine = parts[rank::world]
    circuits = [(api.CuMetaBitsProbCircuit(fc, dev.index), api.DeviceData(data, dev)) for data, fc in mine]
    streams = [torch.cuda.Stream(device=dev) for _ in circuits]
    rng = np.random.default_rng(7)
    n_total = args.warmup + args.steps
    ids = [[torch.from_numpy((rng.permutation(20000)[:B] + 1).astype(np.int32)).to(dev) for _ in circuits] for _ in range(n_total)]
    lls = [torch.zeros(1, device=dev) for _ in circuits]

    def step(i):
        cur = torch.cuda.current_stream(dev)
        for j, (m, dd) in enumerate(circuits):
            streams[j].wait_stream(cur)
            with torch.cuda.stream(streams[j]):
                api.em_step(m, dd, ids[i][j], 1, B, PSEUDOCOUNT, INERTIA, 0.0, None, lls[j])
        for st_ in streams:
            cur.wait_stream(st_)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for i in range(args.warmup):
        step(i)
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(dev.index) as clocks:
        e0.record()
        for i in range(args.warmup, n_total):
            step(i)
        e1.record()
        barrier()
    ms = e0.elapsed_time(e1)
    t = torch.tensor([ms], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item())
    launches = sum(sum(v[1] for v in m.profile_read(reset=True).values()) for m, _ in circuits)
    if rank == 0:
        fc0 = mine[0][1]
        line = {"metric": "samples/sec fwd+bwd+EM", "value": 64 * B * args.steps / (ms * 1e-3), "unit": "samples/s",
                "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms / args.steps,
                "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
                "config": {"workload": "config 3: 64 patch HCLTs (192 vars x 256 cats, 128 latents), B=256 images per circuit, all circuits per step",
                           "circuits": 64, "circuits_per_rank": len(mine), "nodes_per_circuit": fc0.num_nodes,
                           "edges_per_circuit": fc0.num_edges, "parallelism": f"circuits over {world} rank(s), no collective"},
                "train_ll_circuit0": float(lls[0].item()) / B, "clocks": clocks.summary(), "gpu_launches": int(launches)}
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--config", default=os.environ.get("PCB_BENCH_CONFIG", "cfg5"))
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--cpu-seconds", type=float, default=20.0, help="CPU time the cpu_baseline leg of the N=1 run may take")
    ap.add_argument("--reference-seconds", type=float, default=200.0,
                    help="--impl reference: CPU time for all warm-up and timed steps together")
    ap.add_argument("--no-also", action="store_true", help="skip the config 2 / config 4 side measurements of the N=1 run")
    ap.add_argument("--no-weak", action="store_true", help="N > 1: skip the fixed-batch-per-GPU measurement")
    ap.add_argument("--no-parity", action="store_true", help="N>1: skip the comparison with a 1-GPU run of the same steps")
    ap.add_argument("--scaling", default="strong", choices=["strong", "weak"],
                    help="strong: the config's global batch is split over the GPUs (config 5 as stated); "
                         "weak: every GPU takes the config's batch")
    args = ap.parse_args()
    if args.config == "cfg3":
        run_cfg3(args)
        return
    if args.config == "cfg4":
        if int(os.environ.get("RANK", "0")) == 0:
            print(json.dumps(measure_cfg4(args)))
        return
    cfg = CONFIGS[args.config]
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    Bg = cfg["batch"] * (int(os.environ.get("WORLD_SIZE", "1")) if args.scaling == "weak" else 1)

    if args.impl == "reference":
        # The reference has no CPU implementation of this path and Julia is not installed: the
        # CPU arm is the oracle, a C restatement of the reference's kernels, on all host threads.
        if rank != 0:
            return
        import torch
        images, fc = build_workload(cfg, "cuda" if torch.cuda.is_available() else "cpu")
        images_cpu = images[:4096].cpu().numpy()
        del images
        cpu = CpuOracle(fc, images_cpu)
        n_total = args.warmup + args.steps
        # every step is a bounded sample: the rows per step are sized from a first step of one row
        # per thread so that warm-up + timed steps end within about --reference-seconds
        rows, t_e, t_m = cpu.step(cpu.threads)
        per_step = args.reference_seconds / max(1, n_total)
        rows_per_step = int(max(1, min(cfg["batch"], (per_step - t_m) / max(t_e / rows, 1e-9))))
        rows_per_step = max(cpu.threads, rows_per_step // cpu.threads * cpu.threads) if rows_per_step >= cpu.threads else rows_per_step
        meas = []
        for i in range(n_total):
            r = cpu.step(rows_per_step, first_row=(i * rows_per_step) % max(1, images_cpu.shape[0] - rows_per_step))
            if i >= args.warmup:
                meas.append(r)
        rows = meas[0][0]
        t_e, t_m = float(np.mean([x[1] for x in meas])), float(np.mean([x[2] for x in meas]))
        desc = cpu.describe(cfg["batch"], rows, t_e, t_m)
        value = desc["value"]
        line = {"impl": "reference", "metric": "samples/sec fwd+bwd+EM", "value": value, "unit": "samples/s",
                "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
                "ms_per_step": cfg["batch"] / value * 1e3, "measured_ms_per_sample_step": (t_e + t_m) * 1e3,
                "higher_is_better": True,
                "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
                "config": {"workload": cfg["desc"], "bench_config": args.config, "global_batch": cfg["batch"],
                           "parallelism": f"cpu-threads x{cpu.threads}", "rows_per_step": rows},
                "cpu_baseline": desc,
                "e2e": {"value": value, "unit": "samples/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
        print(json.dumps(line))
        return

    import torch
    import torch.distributed as dist
    from lvd_pg_b200 import api

    assert torch.cuda.is_available(), "bench.py needs a CUDA device (no CPU fallback)"
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    assert Bg % world == 0
    B = Bg // world

    t_setup = time.perf_counter()
    images, fc = build_workload(cfg, dev)
    m = api.CuMetaBitsProbCircuit(fc, local_rank)
    data = api.DeviceData(images, dev)
    if world > 1:
        obj = [api.comm_unique_id() if rank == 0 else None]
        dist.broadcast_object_list(obj, src=0)
        m.attach_comm(obj[0], rank, world)
    rows = data.num_rows
    rng = np.random.default_rng(123)
    n_steps_total = args.warmup + args.steps
    perms = [torch.from_numpy((rng.permutation(rows)[:Bg] + 1).astype(np.int32)) for _ in range(n_steps_total)]
    ids = [p[rank * B:(rank + 1) * B].to(dev) for p in perms]
    ll = torch.zeros(1, device=dev)
    p_init = None
    if world > 1 and not args.no_parity:   # the parameters every later comparison starts from
        p_init = api.vectorize_parameters(m, torch.empty(api.num_parameters(m), dtype=torch.float32, device=dev)).clone()
    torch.cuda.synchronize()
    setup_s = time.perf_counter() - t_setup

    def step(i):
        api.em_step(m, data, ids[i], 1, B, PSEUDOCOUNT, INERTIA, 0.0, None, ll)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    clocks = ClockSampler(local_rank, enabled=(rank == 0)).start()   # up before the warm-up, one per job
    for i in range(args.warmup):
        step(i)
    m.profile_read(reset=True)
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    clocks.begin()
    e0.record()
    for i in range(args.warmup, n_steps_total):
        step(i)
    e1.record()
    barrier()
    clocks.end()
    ms = e0.elapsed_time(e1)
    launches = sum(v[1] for v in m.profile_read(reset=True).values())
    t = torch.tensor([ms], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item())
    value = Bg * args.steps / (ms * 1e-3)
    ll_last = float(ll.item()) / Bg   # the statistics vector (and its log-likelihood slot) is summed over ranks

    # ---- per-kernel-class timing (separate pass, events around every launch) -------------------
    m.profile_enable(True)
    prof_steps = 2
    for i in range(prof_steps):
        step(args.warmup + i % max(1, args.steps))
    prof = m.profile_read(reset=True)
    m.profile_enable(False)
    peaks = measured_peaks()
    work = algorithmic_work(fc, m.info, B)
    classes = {k: v for k, v in prof.items() if v[1] > 0}
    total_prof_ms = sum(v[0] for v in classes.values())
    dom = max(classes, key=lambda k: classes[k][0])
    dom_ms = classes[dom][0] / prof_steps
    w = work.get(dom, {})
    if "flops" in w:
        # dense blocks: 2*B*k*k flops over 4*(3..6)*B*k bytes per block is k/6 .. k/12 flops per byte
        # (21 .. 43 at k = 256, three times that with the TF32 passes counted): far under the ridge of
        # the machine, so the HBM roof is the one that binds.  The tensor-pipe view is kept beside it.
        tfl = w["flops"] / (dom_ms * 1e-3) / 1e12
        achieved = w["bytes"] / (dom_ms * 1e-3) / 1e9
        roof = {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                "frac": achieved / peaks["hbm_gbs"], "traffic": None,
                "tensor_view": {"achieved": tfl, "peak": peaks["tflops"], "unit": "TFLOP/s", "frac": tfl / peaks["tflops"],
                                "note": "algorithmic flops 2*B*E_d of the class; the three TF32 passes are not counted"}}
    else:
        achieved = w.get("bytes", 0.0) / (dom_ms * 1e-3) / 1e9
        roof = {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                "frac": achieved / peaks["hbm_gbs"], "traffic": None}
    # the whole step against the HBM roof: algorithmic bytes of every class / timed step
    step_bytes = sum(v.get("bytes", 0.0) for kk, v in work.items() if kk in classes)
    roof["step_hbm"] = {"bytes_per_step": step_bytes, "achieved": step_bytes / (ms / args.steps * 1e-3) / 1e9,
                        "unit": "GB/s", "frac": step_bytes / (ms / args.steps * 1e-3) / 1e9 / peaks["hbm_gbs"]}
    lps = classes[dom][1] / prof_steps
    roof["traffic"] = measured_traffic(dom, m.info, B, lps)
    if roof["traffic"] is not None:
        roof["traffic_unit"] = "bytes per launch (ncu capture of the reduced workload, scaled by blocks x examples)"
        roof["algorithmic_bytes_per_launch"] = w.get("bytes", 0.0) / lps
    # every class against the HBM roof, from its algorithmic bytes and its own event time
    roof["class_hbm_frac"] = {kk: round(work[kk]["bytes"] / (classes[kk][0] / prof_steps * 1e-3) / 1e9 / peaks["hbm_gbs"], 4)
                              for kk in classes if kk in work and classes[kk][0] > 0}
    roof.update({"kernel": dom, "kernel_ms_per_step": dom_ms, "launches_per_step": classes[dom][1] / prof_steps,
                 "peak_source": peaks["which"],
                 "class_ms_per_step": {k: round(v[0] / prof_steps, 4) for k, v in classes.items()},
                 "class_share": {k: round(v[0] / total_prof_ms, 4) for k, v in classes.items()}})

    # ---- end to end: host batches in, log-likelihood out ------------------------------------------
    e2e = None
    if not args.no_e2e:
        images_cpu_rows = images.cpu()
        host_batches = []
        for i in range(n_steps_total):
            sel = (perms[i][rank * B:(rank + 1) * B].long() - 1)
            host_batches.append(images_cpu_rows[sel].t().contiguous().pin_memory())  # [V, B] column-major batch
        del images_cpu_rows
        lls = []

        def e2e_step(i):
            batch = host_batches[i].to(dev, non_blocking=True)
            d = api.DeviceData.from_colmajor(batch)
            api.em_step(m, d, None, 1, B, PSEUDOCOUNT, INERTIA, 0.0, None, ll)
            lls.append(float(ll.item()))  # device -> host read of the step's result

        for i in range(args.warmup):
            e2e_step(i)
        barrier()
        t0 = time.perf_counter()
        for i in range(args.warmup, n_steps_total):
            e2e_step(i)
        barrier()
        dt = time.perf_counter() - t0
        tt = torch.tensor([dt], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        e2e = {"value": Bg * args.steps / float(tt.item()), "unit": "samples/s",
               "h2d_bytes_per_step": int(B * fc.num_vars * world), "d2h_bytes_per_step": 4 * world}

    # ---- N > 1: what the collectives leave exposed, and the same ranks at a fixed batch per GPU -------
    comm = None
    weak = None
    if world > 1:
        def timed(fn, k):
            for i in range(4):   # a changed step takes up to three calls to be captured and replayed again
                fn(i)
            barrier()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            for i in range(k):
                fn(args.warmup + i % max(1, args.steps))
            b.record()
            barrier()
            tt = torch.tensor([a.elapsed_time(b) / k], device=dev, dtype=torch.float64)
            dist.all_reduce(tt, op=dist.ReduceOp.MAX)
            return float(tt.item())

        k_c = min(args.steps, 5)
        with_comm = timed(step, k_c)
        m.lib.pcb_comm_set_enabled(m.handle, 0)      # the same steps, every rank on its own statistics
        without = timed(step, k_c)
        m.lib.pcb_comm_set_enabled(m.handle, 1)
        comm = {"exposed_comm_ms": with_comm - without, "ms_per_step_with": with_comm, "ms_per_step_without": without,
                "allreduce_bytes": 4 * (int(m.info.num_inner_params) + fc.num_input_params + 1),
                "steps": k_c, "how": "device time of the same steps with the collectives skipped, max over ranks"}
        if not args.no_weak:
            # weak scaling beside the strong headline: every rank keeps the configuration's full batch
            ids_w = [p.to(dev) if rank == 0 else torch.roll(p, 97 * rank).to(dev) for p in perms[:args.warmup + max(1, args.steps)]]

            def step_w(i):
                api.em_step(m, data, ids_w[i], 1, Bg, PSEUDOCOUNT, INERTIA, 0.0, None, ll)

            ms_w = timed(step_w, k_c)
            weak = {"scaling": "weak", "global_batch": Bg * world, "ms_per_step": ms_w,
                    "value": Bg * world / (ms_w * 1e-3), "unit": "samples/s", "steps": k_c}
            del ids_w

    # ---- N > 1: the same steps on one GPU with the whole batch, from the same parameters ------------
    parity = None
    if p_init is not None:
        k_par = min(3, n_steps_total)

        def run_steps(shard):
            api.update_parameters(m, p_init)
            out = []
            for i in range(k_par):
                sel = perms[i][rank * B:(rank + 1) * B] if shard else perms[i]
                api.em_step(m, data, sel.to(dev), 1, int(sel.numel()), PSEUDOCOUNT, INERTIA, 0.0, None, ll)
                out.append(float(ll.item()))
            return out, api.vectorize_parameters(m, torch.empty_like(p_init)).clone()

        ll_n, p_n = run_steps(True)
        # every rank must hold the same parameters bit for bit after the replicated update
        p0 = p_n.clone()
        dist.broadcast(p0, src=0)
        same = torch.tensor([1.0 if torch.equal(p0, p_n) else 0.0], device=dev)
        dist.all_reduce(same, op=dist.ReduceOp.MIN)
        del p0
        barrier()
        m.detach_comm()
        if rank == 0:
            ll_1, p_1 = run_steps(False)
            parity = {"steps": k_par, "max_abs_dprob": float((p_n.double().exp() - p_1.double().exp()).abs().max().item()),
                      "ll_rel": max(abs(a - b) / abs(b) for a, b in zip(ll_n, ll_1)),
                      "ranks_bit_identical": bool(same.item() == 1.0)}
            parity["ok"] = bool(parity["max_abs_dprob"] <= 1e-4 and parity["ll_rel"] <= 1e-4 and parity["ranks_bit_identical"])
        barrier()

    cpu_baseline = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        cpu = CpuOracle(fc, images[:4096].cpu().numpy())
        # at least 64 rows (four per thread on a 16-thread host), more while the leg stays inside --cpu-seconds
        r0, te0, tm0 = cpu.step(cpu.threads)
        want = int((args.cpu_seconds - tm0) / max(te0 / r0, 1e-9))
        rows_c = max(64, min(cfg["batch"], want // cpu.threads * cpu.threads))
        r1, te1, tm1 = cpu.step(rows_c, first_row=r0)
        cpu_baseline = cpu.describe(cfg["batch"], r1, te1, tm1)
        del cpu

    if rank == 0:
        n_edges = fc.num_edges
        line = {"metric": "samples/sec fwd+bwd+EM", "value": value, "unit": "samples/s", "n_gpus": world,
                "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True,
                "scaling": args.scaling, "vs_baseline": None, "dtype": "f32", "data": "synthetic",
                "config": {"workload": cfg["desc"], "bench_config": args.config, "global_batch": Bg,
                           "parallelism": f"dp{world}", "l2": "inputs (mars+flows) larger than L2" if
                           fc.num_nodes * B * 8 > 126e6 else "working set below L2",
                           "nodes": fc.num_nodes, "edges": n_edges, "sum_edges": int(m.info.num_inner_params),
                           "dense_blocks": int(m.info.num_dense_blocks), "up_layers": int(m.info.num_up_layers),
                           "leaf_params": fc.num_input_params, "setup_s": round(setup_s, 1)},
                "edges_samples_per_s": value * n_edges, "train_ll_last_batch": ll_last,
                "clocks": clocks.summary(), "gpu_launches": int(launches), "roofline": roof}
        if e2e:
            line["e2e"] = e2e
        if cpu_baseline:
            line["cpu_baseline"] = cpu_baseline
        if parity:
            line["parity_vs_1gpu"] = parity
        if comm:
            line["exposed_comm_ms"] = comm["exposed_comm_ms"]
            line["comm"] = comm
        if weak:
            line["weak"] = weak
        if world == 1 and not args.no_also and args.config == "cfg5":
            # the other configurations' headline figures, measured in the same run (a second of GPU time each)
            del m, data, images
            torch.cuda.empty_cache()
            also = {}
            try:
                also["cfg2"] = measure_cfg2_step()
                torch.cuda.empty_cache()
                c4 = measure_cfg4(argparse.Namespace(steps=20, warmup=5, no_cpu_baseline=True), cpu_leg=False)
                also["cfg4"] = {"workload": c4["config"]["workload"], "us_per_kld_grad_adam_step": c4["value"],
                                "hard_samples_per_s": c4["sampling"]["samples_per_s"], "hard_sampling_ms_per_call": c4["sampling"]["ms_per_call"]}
            except Exception as e:   # a side measurement must not lose the headline line
                also["error"] = repr(e)
            line["also"] = also
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
