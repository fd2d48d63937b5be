"""Benchmark of the VSA forward+backward hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference|reference_triton] [--workload NAME]

One "step" is one forward+backward of the whole operator over this rank's share of
the workload.  The default workload is the 92,160-token / block-64 / topk-180 shape
``[B=2,H=40,L=92160,D=128]`` bf16 with all blocks full; its 80 (batch, head) slices
are partitioned contiguously across the N ranks with no data-path collective (heads
are independent), so total work is fixed and scaling is "strong".  Inputs are
synthetic N(0,1), generated per (batch, head) slice from ``seed + slice`` so every
sharding sees identical data.

The JSON line (printed by rank 0) carries: ``value`` = useful sparse TFLOP/s over all
ranks with inputs resident in HBM (useful FLOPs = 14*B*H*L*topk*be*D per call);
``e2e`` = the same through the public API with pinned host buffers copied in and the
results copied out inside the timed region; ``roofline`` for the dominant kernel
from CUDA events recorded around every launch of the timed steps; ``cpu_baseline``
= the reference's own ``vsa.torch_vsa`` (installed copy under ``baseline/_ref``; the
oracle port when that copy is absent) timed on a bounded sample of the same workload
with all host cores and with one; ``e2e.copy_floor_ms`` = the end-to-end step's copy
schedule with the operator left out; SM clocks sampled during the timed region; and,
at one GPU, ``gpu_reference`` = the installed reference copy's own Triton kernels
timed on the same tensors for the same number of steps.

``--impl reference`` times that CPU implementation alone (rank 0 only under torchrun).
``--impl reference_triton`` (extra) times only the reference copy's Triton kernels.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

WORKLOADS = {
    # name: (B, H, L, D, block_size, topk, gate, ragged)
    "c5_92k_be64_tk180": dict(B=2, H=40, L=92160, D=128, block_size=(4, 4, 4), topk=180, gate=False),
    "c2_16k_be64_tk32_gate": dict(B=1, H=12, L=16384, D=128, block_size=(4, 4, 4), topk=32, gate=True),
    # one tenth of the headline slices, with a gate: the profiling case (2.8 GB on the device, tensors > L2)
    "mid_92k_h8_tk180_gate": dict(B=1, H=8, L=92160, D=128, block_size=(4, 4, 4), topk=180, gate=True),
    # two slices of the headline shape: small enough for multi-pass ncu captures (0.4 GB of tensors + 4.2 GB dS workspace)
    "prof_92k_h2_tk180": dict(B=1, H=2, L=92160, D=128, block_size=(4, 4, 4), topk=180, gate=False),
    "small_8k_be64_tk16": dict(B=1, H=8, L=8192, D=128, block_size=(4, 4, 4), topk=16, gate=False),
    # logical 256 blocks, 10 % of them ragged (sizes uniform in [1,255], padded rows zeroed)
    "c3_40k_be256_tk20_ragged": dict(B=1, H=40, L=40960, D=128, block_size=(4, 8, 8), topk=20, gate=False,
                                     ragged_frac=0.1),
    # sequence-parallel long-sequence run: every rank owns L/W query tokens and the matching K/V shard,
    # K/V are all-gathered over NCCL, dK/dV reduce-scattered (weak in L per rank is NOT assumed: L is fixed)
    "c5sp_184k_be64_tk360": dict(B=2, H=40, L=184320, D=128, block_size=(4, 4, 4), topk=360, gate=False, sp=True),
    "sp_small_32k_be64_tk64": dict(B=1, H=8, L=32768, D=128, block_size=(4, 4, 4), topk=64, gate=False, sp=True),
    # route-explicit executor only: 180 of 1440 key blocks per query block, Zipf(1.1) without replacement
    "c4_92k_routes_zipf": dict(B=1, H=40, L=92160, D=128, block_size=(4, 4, 4), topk=180, gate=False, routes="zipf"),
    # the three route kinds of the reference's component bench (examples/bench_components.py:51-63) at the same shape:
    # uniform = Top-K of random scores, local = the next topk blocks (mod Kb), hotset = every query block reads blocks 0..topk-1
    "c4_92k_routes_uniform": dict(B=1, H=40, L=92160, D=128, block_size=(4, 4, 4), topk=180, gate=False, routes="uniform"),
    "c4_92k_routes_local": dict(B=1, H=40, L=92160, D=128, block_size=(4, 4, 4), topk=180, gate=False, routes="local"),
    "c4_92k_routes_hotset": dict(B=1, H=40, L=92160, D=128, block_size=(4, 4, 4), topk=180, gate=False, routes="hotset"),
    # the reference's own CPU-runnable case: fp32, 16 full blocks of 64, head dim 64, topk 4 (fp32 runs on the CUDA-core kernels)
    # the profiling case with blocks of 128 tokens (two 64-token tiles per block), same useful FLOPs as be 64 / topk 180
    "mid_92k_h8_be128_tk90_gate": dict(B=1, H=8, L=92160, D=128, block_size=(4, 4, 8), topk=90, gate=True),
    # c2 at head dim 64: the warp-level (mma.sync) tensor-core kernels; VSA_B200_KERNELS=scalar times the CUDA-core ones
    "c2_d64_16k_be64_tk32_gate": dict(B=1, H=12, L=16384, D=64, block_size=(4, 4, 4), topk=32, gate=True),
    # the profiling case in fp16: the same tcgen05 kernels instantiated for the other 16-bit input format
    "mid_92k_h8_tk180_gate_fp16": dict(B=1, H=8, L=92160, D=128, block_size=(4, 4, 4), topk=180, gate=True, dtype="f16"),
    "c1_1k_be64_tk4_fp32": dict(B=1, H=2, L=1024, D=64, block_size=(1, 1, 64), topk=4, gate=False, dtype="f32"),
}
DEFAULT_WORKLOAD = "c5_92k_be64_tk180"
SEED = 1234


def useful_flops(slices: int, L: int, topk: int, be: int, D: int) -> float:
    """fwd 4*be^2*D + bwd 10*be^2*D per (query block, key block) edge."""
    return 14.0 * slices * L * topk * be * D


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as fh:
            p = json.load(fh)
        return dict(tflops=float(p.get("bf16_tflops_sustained", p.get("bf16_tflops"))), hbm=float(p["hbm_gbs"]),
                    source="measured (MEASURED_PEAKS.json, sustained bf16)")
    return dict(tflops=1590.0, hbm=6650.0, source="fallback (no MEASURED_PEAKS.json: 1590 TFLOP/s bf16, 6650 GB/s)")


# --------------------------------------------------------------------------------------------
# clocks
# --------------------------------------------------------------------------------------------
class ClockSampler:
    """Samples nvidia-smi every 200 ms while the timed region runs."""

    FIELDS = ("index,clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap,power.draw")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "200",
                 "-i", str(self.gpu)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._pump, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, watts, reasons = [], [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[1]))
                mx.append(float(parts[2]))
            except ValueError:
                continue
            for name, val in zip(names, parts[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(name)
            if len(parts) > 7:
                try:
                    watts.append(float(parts[7]))
                except ValueError:
                    pass
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons),
                "power_w": statistics.median(watts) if watts else None}


# --------------------------------------------------------------------------------------------
# CPU arm (oracle port of the reference algorithm on a bounded sample)
# --------------------------------------------------------------------------------------------
def _reference_torch_vsa():
    """``vsa.torch_vsa`` of the UNMODIFIED reference package installed under ``baseline/_ref`` (pure PyTorch), or
    None when that copy is absent or does not import."""
    ref_dir = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref_dir, "vsa")):
        return None
    if ref_dir not in sys.path:
        sys.path.insert(0, ref_dir)
    try:
        from vsa.torch_impl import torch_vsa
        return torch_vsa
    except Exception:       # noqa: BLE001 - any import problem falls back to the port
        return None


def cpu_sample_setup(cfg, q_blocks: int):
    """One (batch, head) slice of the workload: full-length K/V, the first ``q_blocks`` query blocks.

    The timed code is the reference's own ``torch_vsa`` (``vsa/torch_impl.py:49-113``) when the installed copy
    imports -- it accepts fewer query tokens than key tokens, so the sample is a plain call of it -- and the
    oracle port of the same algorithm otherwise.  Small workloads (the reference's CPU case) run whole.
    """
    import torch
    from oracle import vsa_oracle as O

    be = O.block_elements(cfg["block_size"])
    L, D, tk = cfg["L"], cfg["D"], cfg["topk"]
    dt = workload_dtype(cfg)
    whole = cfg["B"] * cfg["H"] * (L // be) <= 64
    slices = cfg["B"] * cfg["H"] if whole else 1
    q_blocks = L // be if whole else min(q_blocks, L // be)
    g = torch.Generator().manual_seed(SEED)
    q = torch.randn(1, slices, q_blocks * be, D, generator=g).to(dt)
    k = torch.randn(1, slices, L, D, generator=g).to(dt)
    v = torch.randn(1, slices, L, D, generator=g).to(dt)
    sizes = torch.full((L // be,), be)
    q_sizes = torch.full((q_blocks,), be)
    dout = torch.randn(1, slices, q_blocks * be, D, generator=g).to(dt)
    ref = _reference_torch_vsa()

    def step():
        ql, kl, vl = q.clone().requires_grad_(), k.clone().requires_grad_(), v.clone().requires_grad_()
        if ref is not None:
            out = ref(ql, kl, vl, sizes, q_sizes, tk, cfg["block_size"], None)
        else:
            out = O.vsa(ql, kl, vl, sizes, q_sizes, tk, cfg["block_size"], None, q_blocks_per_chunk=8)
        out.backward(dout)
        return out

    flops = useful_flops(slices, q_blocks * be, tk, be, D)
    what = "the reference's own vsa.torch_vsa (installed copy under baseline/_ref)" if ref is not None else \
        "oracle port (CPU restatement of torch_vsa)"
    sample = (f"{what}: " + ("the whole workload" if whole else
              f"1 of {cfg['B'] * cfg['H']} (batch,head) slices, the first {q_blocks} of {L // be} query blocks "
              f"against all {L // be} key blocks") +
              f" (topk {tk}, block {be}, D {D}, {'fp32' if dt == torch.float32 else dtype_name(cfg) + ' inputs, fp32 fine math'}), "
              "forward+backward; throughput = the sample's useful FLOPs / its time")
    return step, flops, sample, ("reference" if ref is not None else "port")


def run_cpu(cfg, steps: int, warmup: int, q_blocks: int = 16):
    """Times the CPU sample with every core this process may use, and once more on one thread."""
    import torch
    cores = len(os.sched_getaffinity(0))
    torch.set_num_threads(cores)        # torch.distributed.run exports OMP_NUM_THREADS=1: do not inherit that
    step, flops, sample, kind = cpu_sample_setup(cfg, q_blocks)
    for _ in range(warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(steps):
        step()
    dt = (time.perf_counter() - t0) / max(1, steps)
    torch.set_num_threads(1)
    step()
    t0 = time.perf_counter()
    step()
    dt1 = time.perf_counter() - t0
    torch.set_num_threads(cores)
    return dict(value=flops / dt / 1e12, unit="TFLOP/s", cores=cores, kind=kind, sample=sample,
                ms_per_step=dt * 1e3, one_thread_value=flops / dt1 / 1e12, one_thread_ms_per_step=dt1 * 1e3)


# --------------------------------------------------------------------------------------------
# GPU arm
# --------------------------------------------------------------------------------------------
def workload_dtype(cfg):
    import torch
    return {"f32": torch.float32, "f16": torch.float16}.get(cfg.get("dtype"), torch.bfloat16)


def dtype_name(cfg):
    return cfg.get("dtype", "bf16")


def make_slices(cfg, first: int, count: int, device, rows=None, salt: int = 0):
    """q, k, v, dout (and gate) for ``count`` (batch, head) slices starting at ``first``: [1, count, rows, D]."""
    import torch
    L, D = (rows or cfg["L"]), cfg["D"]
    names = ["q", "k", "v", "dout"] + (["gate"] if cfg["gate"] else [])
    dt = workload_dtype(cfg)
    out = {n: torch.empty((1, count, L, D), device=device, dtype=dt) for n in names}
    gen = torch.Generator(device=device)
    for i in range(count):
        gen.manual_seed(SEED + first + i + 1000003 * salt)
        for n in names:
            x = torch.randn((L, D), generator=gen, device=device, dtype=torch.float32)
            if n == "gate":
                x = torch.sigmoid(x)
            out[n][0, i] = x.to(dt)
    return out


class KernelTimer:
    """CUDA events around every C-ABI call while enabled (hooked into simple_vsa_b200._lib.call)."""

    def __init__(self):
        import torch
        self.torch = torch
        self.events = {}
        self.pending = {}

    def __call__(self, name, phase, stream):
        ev = self.torch.cuda.Event(enable_timing=True)
        ev.record(self.torch.cuda.current_stream())
        # one name per kernel: the entry points with the block-mean backward folded in, and the shard-major forms of
        # the sequence-parallel mode, launch the same kernels
        name = name.replace("_fused", "").replace("_sharded", "")
        if phase == "start":
            self.pending[name] = ev
        else:
            self.events.setdefault(name, []).append((self.pending.pop(name), ev))

    def summary(self):
        out = {}
        for name, pairs in self.events.items():
            ms = [a.elapsed_time(b) for a, b in pairs]
            out[name] = dict(launches=len(ms), total_ms=sum(ms), avg_ms=sum(ms) / len(ms))
        return out


def time_reference_triton(inputs, cfg, tk, steps, flops_total, own_ms, gpu_index):
    """The UNMODIFIED reference package's own GPU kernels (``vsa.triton_vsa``, ``vsa/triton_impl.py:1734-1765``, from
    the installed copy under ``baseline/_ref``) on the tensors this run has just used: same call, same step count,
    CUDA events (the method of ``examples/bench_full.py:36-48``), clocks sampled alongside."""
    ref_dir = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref_dir, "vsa")):
        return {"impl": "reference_triton", "unavailable": "baseline/_ref holds no installed copy of the reference"}
    if ref_dir not in sys.path:
        sys.path.insert(0, ref_dir)
    try:
        import torch
        from vsa import triton_vsa
        q, k, v = (inputs[n].clone().requires_grad_() for n in ("q", "k", "v"))
        gate, dout = inputs["gate"], inputs["dout"]
        sizes = inputs["sizes"].to(torch.int64)

        def step():
            q.grad = k.grad = v.grad = None
            triton_vsa(q, k, v, sizes, sizes, tk, cfg["block_size"], gate).backward(dout)

        for _ in range(2):
            step()
        torch.cuda.synchronize()
        sampler = ClockSampler(gpu_index)
        sampler.start()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            step()
        e1.record()
        torch.cuda.synchronize()
        clocks = sampler.stop()
        ms = e0.elapsed_time(e1) / steps
        return {"impl": "reference_triton", "ms_per_step": ms, "value": flops_total / (ms * 1e-3) / 1e12,
                "unit": "TFLOP/s", "steps": steps, "clocks": clocks, "speedup": ms / own_ms,
                "what": "vsa.triton_vsa of the installed reference copy, same tensors and step count, this GPU"}
    except Exception as exc:        # noqa: BLE001 - reported, not raised: this leg is a comparison, not the product
        return {"impl": "reference_triton", "unavailable": f"{type(exc).__name__}: {exc}"[:300]}


def run_gpu(args, cfg, rank: int, world: int, local_rank: int):
    import torch
    import torch.distributed as dist

    import simple_vsa_b200 as V
    from simple_vsa_b200 import _lib
    from simple_vsa_b200.parallel import sequence_parallel_vsa

    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    from simple_vsa_b200.host import bind_to_gpu_numa_node
    numa_node = bind_to_gpu_numa_node(local_rank)      # before any pinned host memory is allocated
    if world > 1:
        opts = None
        try:        # NCCL's kernels on a high-priority stream: they must find SMs between our long one-CTA-per-SM kernels
            opts = dist.ProcessGroupNCCL.Options(is_high_priority_stream=True)
        except Exception:       # noqa: BLE001 - older builds: default options
            opts = None
        dist.init_process_group("nccl", device_id=dev, pg_options=opts)
    be = V.as_block_elements(cfg["block_size"])
    L, D, tk = cfg["L"], cfg["D"], cfg["topk"]
    total_slices = cfg["B"] * cfg["H"]
    sp = bool(cfg.get("sp"))
    per = total_slices // world
    extra = total_slices % world
    count = per + (1 if rank < extra else 0)
    first = rank * per + min(rank, extra)
    sizes = torch.full((L // be,), be, dtype=torch.int32, device=dev)
    nb = L // be
    if sp:      # every rank holds all slices but only L/W tokens (its query blocks and its K/V shard)
        if L % (world * be):
            raise SystemExit(f"sequence-parallel workload needs L divisible by world*block ({world}*{be})")
        count, first = total_slices, 0
    l_loc = L // world if sp else L

    data = make_slices(cfg, first, count, dev, rows=l_loc, salt=rank if sp else 0)
    q, k, v, dout = data["q"], data["k"], data["v"], data["dout"]
    gate = data.get("gate")
    if cfg.get("ragged_frac"):
        g = torch.Generator().manual_seed(SEED)
        ragged = torch.randperm(nb, generator=g)[:max(1, int(round(nb * cfg["ragged_frac"])))]
        sizes_h = torch.full((nb,), be, dtype=torch.int32)
        sizes_h[ragged] = torch.randint(1, be, (ragged.numel(),), generator=g, dtype=torch.int32)
        sizes = sizes_h.to(dev)
        pad = (torch.arange(be)[None, :] >= sizes_h[:, None]).reshape(L).to(dev)      # [L] True on padding rows
        for t in (q, k, v):
            t[:, :, pad] = 0
    routes = None
    if cfg.get("routes") in ("uniform", "local", "hotset"):
        # the generators of the reference's component bench (examples/bench_components.py:51-63)
        if cfg["routes"] == "uniform":
            gen = torch.Generator(device=dev)
            routes = torch.empty((1, count, nb, tk), device=dev, dtype=torch.int32)
            for i in range(count):
                gen.manual_seed(SEED + 7919 * (first + i))
                routes[0, i] = torch.randn((nb, nb), generator=gen, device=dev).topk(tk, dim=-1).indices.to(torch.int32)
        else:
            qi = torch.arange(nb, device=dev)[:, None]
            slots = torch.arange(tk, device=dev)[None, :]
            one = (qi + slots) % nb if cfg["routes"] == "local" else slots.expand(nb, -1)
            routes = one[None, None].expand(1, count, -1, -1).to(torch.int32).contiguous()
    elif cfg.get("routes") == "zipf":
        gen = torch.Generator(device=dev)
        routes = torch.empty((1, count, nb, tk), device=dev, dtype=torch.int32)
        logw = -1.1 * torch.log(torch.arange(1, nb + 1, device=dev, dtype=torch.float32))
        for i in range(count):
            gen.manual_seed(SEED + 7919 * (first + i))
            perm = torch.randperm(nb, generator=gen, device=dev)
            u = torch.rand((nb, nb), generator=gen, device=dev).clamp_min(1e-12)
            routes[0, i] = perm[(logw - torch.log(-torch.log(u))).topk(tk, dim=-1).indices].to(torch.int32)
        del u

    def fwd_bwd(q_, k_, v_, gate_, dout_):
        q_.grad = k_.grad = v_.grad = None
        if gate_ is not None:
            gate_.grad = None
        if sp:
            out = sequence_parallel_vsa(q_, k_, v_, sizes, sizes[:l_loc // be], tk, cfg["block_size"], gate_)
        elif routes is not None:
            out = V.b200_sparse_attention(q_, k_, v_, routes, sizes, block_size=cfg["block_size"])
        else:
            out = V.b200_vsa(q_, k_, v_, sizes, sizes, tk, cfg["block_size"], gate_)
        out.backward(dout_)
        return out

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    leaves = [t.requires_grad_() for t in (q, k, v)]
    gl = gate.requires_grad_() if gate is not None else None
    for _ in range(args.warmup):
        fwd_bwd(*leaves, gl, dout)
    barrier()

    # ---- device-resident timing, every kernel bracketed by events ----
    timer = KernelTimer()
    sampler = ClockSampler(local_rank)
    launches_before = _lib.lib.vsa_launch_count()
    if rank == 0:
        sampler.start()
    _lib.recorder = timer
    barrier()
    t_start, t_stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t_start.record()
    for _ in range(args.steps):
        fwd_bwd(*leaves, gl, dout)
    t_stop.record()
    barrier()
    _lib.recorder = None
    clocks = sampler.stop() if rank == 0 else None
    launches = _lib.lib.vsa_launch_count() - launches_before
    ms_dev = t_start.elapsed_time(t_stop) / args.steps
    kernels = timer.summary()
    _lib.raise_on_device_timeout("bench (timed steps)")      # a drained kernel must not pass for a fast one

    # ---- end to end: pinned host buffers in, results out, inside the timed region ----
    names = ["q", "k", "v", "dout"] + (["gate"] if gate is not None else [])
    dt = workload_dtype(cfg)
    host_in = {n: torch.empty(data[n].shape, dtype=dt, pin_memory=True) for n in names}
    for n in names:
        host_in[n].copy_(data[n].detach())
    out_names = ["out", "dq", "dk", "dv"] + (["dgate"] if gate is not None else [])
    host_out = {n: torch.empty(q.shape, dtype=dt, pin_memory=True) for n in out_names}
    ref_inputs = None
    if world == 1 and not args.no_gpu_reference and not sp and routes is None:
        ref_inputs = dict(q=q.detach(), k=k.detach(), v=v.detach(), dout=dout, gate=None if gate is None else gate.detach(),
                          sizes=sizes)
    del data, q, k, v, dout, gate, leaves, gl
    torch.cuda.empty_cache()
    e2e_steps = max(1, args.steps if args.e2e_steps is None else args.e2e_steps)

    from simple_vsa_b200.host import vsa_step_from_host

    pipelined = routes is None and not sp

    def e2e_step(copy_schedule_only=False):
        if not pipelined:     # route-explicit executor / sequence-parallel: plain copy in / call / copy out
            dv_ = {n: host_in[n].to(dev, non_blocking=True) for n in names}
            if copy_schedule_only:
                for n, src in zip(("out", "dq", "dk", "dv"), ("q", "k", "v", "dout")):
                    host_out[n].copy_(dv_[src], non_blocking=True)
                return
            ql, kl, vl = (dv_[n].requires_grad_() for n in ("q", "k", "v"))
            out = fwd_bwd(ql, kl, vl, None, dv_["dout"])
            for n, t in (("out", out.detach()), ("dq", ql.grad), ("dk", kl.grad), ("dv", vl.grad)):
                host_out[n].copy_(t, non_blocking=True)
            return
        # the public host-resident step: chunks of slices, copies overlapped with the kernels
        vsa_step_from_host(host_in["q"], host_in["k"], host_in["v"], host_in["dout"], sizes, sizes, tk,
                           cfg["block_size"], host_in.get("gate"), out=host_out, device=dev,
                           slices_per_chunk=args.e2e_chunk, copy_schedule_only=copy_schedule_only)

    def timed(fn, n):
        fn()
        barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(n):
            fn()
        b.record()
        barrier()
        return a.elapsed_time(b) / n

    ms_e2e = timed(e2e_step, e2e_steps)
    checksum = float(host_out["out"][0, 0, :64].float().abs().sum())
    _lib.raise_on_device_timeout("bench (end-to-end steps)")
    # the same copies on the same streams with the operator left out: what the transfers alone cost on this machine
    ms_floor = timed(lambda: e2e_step(copy_schedule_only=True), max(1, min(3, e2e_steps)))

    # ---- max over ranks ----
    if world > 1:
        t = torch.tensor([ms_dev, ms_e2e, ms_floor], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_dev, ms_e2e, ms_floor = float(t[0]), float(t[1]), float(t[2])
        lt = torch.tensor([launches], device=dev, dtype=torch.int64)
        dist.all_reduce(lt, op=dist.ReduceOp.SUM)
        launches = int(lt[0])
    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    flops_total = useful_flops(total_slices, L, tk, be, D)
    peaks = measured_peaks()
    # dominant kernel by total device time
    # GEMM FLOPs a kernel's algorithm performs per edge (units of be^2*D): forward S,O = 4; recomputing dQ pass S,dP,dQ = 6;
    # dK/dV pass S,dP,dK,dV = 8 (with or without the dS stores); dQ from stored dS = 2
    gemm_units = {"vsa_sparse_fwd": 4, "vsa_sparse_fwd_combine": 4, "vsa_sparse_bwd_dq": 6, "vsa_sparse_bwd_dkdv": 8, "vsa_sparse_bwd_dkdv_ds": 8,
                  "vsa_sparse_bwd_dq_from_ds": 2}
    fine = {n: kernels[n] for n in gemm_units if n in kernels}
    top = max(fine, key=lambda n: fine[n]["total_ms"])
    per_edge = gemm_units[top]
    # a kernel may be launched several times per step (groups of slices, head groups): its launches of one step
    # together cover every edge of this rank once, so the rate is edges per step over its time per step
    edges = count * (l_loc // be) * tk
    flops_step = per_edge * float(be) * be * D * edges
    top_ms_per_step = fine[top]["total_ms"] / args.steps
    achieved = flops_step / (top_ms_per_step * 1e-3) / 1e12
    traffic = None
    tpath = os.path.join(ROOT, "profiles", "traffic.json")
    if os.path.exists(tpath):
        with open(tpath) as fh:
            tj = json.load(fh)
        if top in tj:
            traffic = tj[top]["dram_bytes_per_tensor_byte"] * count * L * D * 2
    step_total = sum(kv["total_ms"] for kv in kernels.values())
    shares = {n: round(kv["total_ms"] / step_total, 4) for n, kv in sorted(kernels.items())}

    gpu_ref = None
    if ref_inputs is not None:
        gpu_ref = time_reference_triton(ref_inputs, cfg, tk, args.steps, flops_total, ms_dev, local_rank)
        del ref_inputs
    cpu = run_cpu(cfg, steps=args.cpu_steps, warmup=1) if world == 1 and not args.no_cpu else None
    es = 4 if cfg.get("dtype") == "f32" else 2
    T = total_slices * L * D * es          # bytes of one q-shaped tensor over all ranks
    T_rank = count * l_loc * D * es        # ... and on this rank
    n_in, n_out = len(names), len(out_names)
    line = {
        "metric": "VSA fwd+bwd useful TFLOPS, 92k tok blk64 bf16" if args.workload == DEFAULT_WORKLOAD
                  else f"VSA fwd+bwd useful TFLOPS ({args.workload})",
        "value": flops_total / (ms_dev * 1e-3) / 1e12,
        "unit": "TFLOP/s",
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms_dev,
        "higher_is_better": True,
        "scaling": "strong",
        "vs_baseline": None,
        "dtype": dtype_name(cfg),
        "data": "synthetic N(0,1), seeded per (batch,head) slice; random routes come from the operator's own Top-K",
        "collectives": ("all-gather K,V + reduce-scatter dK,dV over NCCL (sequence parallel)" if sp else "none"),
        "config": {"workload": args.workload, "shape_BHLD": [cfg["B"], cfg["H"], L, D], "block_elements": be,
                   "topk": tk, "gate": cfg["gate"], "slices_per_gpu": count, "ragged_frac": cfg.get("ragged_frac", 0),
                   "routes": cfg.get("routes", "operator Top-K"),
                   "parallelism": (f"sequence split over {world} GPU(s): L/W = {l_loc} tokens per rank" if sp else
                                   f"(batch,head) slices partitioned over {world} GPU(s), no collective"),
                   "l2": "inputs per GPU (%.2f GB) are larger than L2; no flush" % (4 * T_rank / 1e9),
                   "useful_flops_per_call": flops_total},
        "impl": "b200",
        "e2e": {"value": flops_total / (ms_e2e * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": ms_e2e,
                "steps": e2e_steps, "h2d_bytes_per_step": n_in * T, "d2h_bytes_per_step": n_out * T,
                "checksum": checksum, "copy_floor_ms": ms_floor,
                "copy_floor_note": "same chunked host<->device copy schedule with the operator left out, max over ranks; "
                                   "the end-to-end step cannot be faster than this on this machine",
                "copy_gbs_per_direction_per_gpu": n_in * T_rank / (ms_floor * 1e-3) / 1e9,
                # what the end-to-end step can at best be: the slower of the device-resident step and the copies alone
                "bound": "host<->device copies" if ms_floor > ms_dev else "kernels",
                "over_bound": ms_e2e / max(ms_floor, ms_dev),
                "numa_node_bound": numa_node},
        "gpu_launches": launches,
        "clocks": clocks,
        "roofline": {"bound": "tensor", "kernel": top, "achieved": achieved, "peak": peaks["tflops"],
                     "unit": "TFLOP/s", "frac": achieved / peaks["tflops"], "traffic": traffic,
                     "peak_source": peaks["source"], "avg_launch_ms": fine[top]["avg_ms"],
                     "launches_per_step": fine[top]["launches"] / args.steps, "ms_per_step": top_ms_per_step,
                     "gemm_flops_per_edge_over_be2D": per_edge,
                     "useful_frac_whole_step": flops_total / world / (ms_dev * 1e-3) / 1e12 / peaks["tflops"]},
        "kernel_time_share": shares,
        "kernel_avg_ms": {n: round(kv["avg_ms"], 4) for n, kv in sorted(kernels.items())},
        "kernel_ms_per_step": {n: round(kv["total_ms"] / args.steps, 4) for n, kv in sorted(kernels.items())},
    }
    if cpu is not None:
        line["cpu_baseline"] = cpu
    if gpu_ref is not None:
        line["gpu_reference"] = gpu_ref
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def run_reference_gpu(args, cfg, rank: int, world: int, local_rank: int):
    """``--impl reference_triton``: the UNMODIFIED reference package (installed by ``__graft_entry__.build()``
    into ``baseline/_ref``, never part of this repository's sources) running its own Triton kernels through its
    own public API on the same GPU, same workload, same synthetic slices, CUDA events.  An extra comparison
    point beside the required CPU reference arm; prints an ``unavailable`` line when the package or Triton
    cannot be imported."""
    def unavailable(why):
        if rank == 0:
            print(json.dumps({"impl": "reference_triton", "unavailable": why}), flush=True)

    ref_dir = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref_dir, "vsa")):
        return unavailable("baseline/_ref is not installed (run __graft_entry__.build() where the reference is present)")
    if cfg.get("sp"):
        return unavailable("the reference has no sequence-parallel mode")
    sys.path.insert(0, ref_dir)
    try:
        import torch
        import torch.distributed as dist
        from vsa import triton_sparse_attention, triton_vsa
    except Exception as exc:        # noqa: BLE001 - any import problem is reported, not raised
        return unavailable(f"import failed: {type(exc).__name__}: {exc}"[:200])
    from oracle.vsa_oracle import block_elements

    if not torch.cuda.is_available():
        return unavailable("no CUDA device")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    be = block_elements(cfg["block_size"])
    L, D, tk = cfg["L"], cfg["D"], cfg["topk"]
    total = cfg["B"] * cfg["H"]
    per, extra = divmod(total, world)
    count, first = per + (1 if rank < extra else 0), rank * per + min(rank, extra)
    nb = L // be
    data = make_slices(cfg, first, count, dev)
    sizes = torch.full((nb,), be, dtype=torch.int64, device=dev)
    if cfg.get("routes"):
        return unavailable("explicit-route workloads are timed for this package only")
    if cfg.get("ragged_frac"):      # the same ragged blocks as run_gpu: seeded choice, sizes in [1, be), padding rows zeroed
        g = torch.Generator().manual_seed(SEED)
        ragged = torch.randperm(nb, generator=g)[:max(1, int(round(nb * cfg["ragged_frac"])))]
        sizes_h = torch.full((nb,), be, dtype=torch.int32)
        sizes_h[ragged] = torch.randint(1, be, (ragged.numel(),), generator=g, dtype=torch.int32)
        sizes = sizes_h.to(dev, torch.int64)
        pad = (torch.arange(be)[None, :] >= sizes_h[:, None]).reshape(L).to(dev)
        for n in ("q", "k", "v"):
            data[n][:, :, pad] = 0
    q, k, v = (data[n].requires_grad_() for n in ("q", "k", "v"))
    gate, dout = data.get("gate"), data["dout"]

    def step():
        q.grad = k.grad = v.grad = None
        out = triton_vsa(q, k, v, sizes, sizes, tk, cfg["block_size"], gate)
        out.backward(dout)
        return out

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(1, args.warmup)):
        step()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        out = step()
    e1.record()
    barrier()
    clocks = sampler.stop() if rank == 0 else None
    ms = e0.elapsed_time(e1) / args.steps
    if world > 1:
        t = torch.tensor([ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t[0])
        dist.destroy_process_group()
    if rank != 0:
        return
    flops_total = useful_flops(total, L, tk, be, D)
    print(json.dumps({
        "metric": "VSA fwd+bwd useful TFLOPS, 92k tok blk64 bf16" if args.workload == DEFAULT_WORKLOAD
                  else f"VSA fwd+bwd useful TFLOPS ({args.workload})",
        "value": flops_total / (ms * 1e-3) / 1e12, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic N(0,1), seeded per (batch,head) slice", "impl": "reference_triton",
        "config": {"workload": args.workload, "shape_BHLD": [cfg["B"], cfg["H"], L, D], "block_elements": be,
                   "topk": tk, "gate": cfg["gate"], "slices_per_gpu": count},
        "e2e": None, "gpu_launches": None, "clocks": clocks,
        "checksum": float(out[0, 0, :64].float().abs().sum())}), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference", "reference_triton"])
    ap.add_argument("--workload", default=DEFAULT_WORKLOAD, choices=sorted(WORKLOADS))
    ap.add_argument("--e2e-steps", type=int, default=None, help="end-to-end steps (default: --steps)")
    ap.add_argument("--cpu-steps", type=int, default=2)
    ap.add_argument("--no-gpu-reference", action="store_true",
                    help="skip timing the installed reference copy's Triton kernels after the own run (1 GPU only)")
    ap.add_argument("--e2e-chunk", type=int, default=8, help="(batch,head) slices per pipelined chunk of the host-resident step")
    ap.add_argument("--no-cpu", action="store_true")
    args = ap.parse_args()
    cfg = WORKLOADS[args.workload]
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))

    if args.impl == "reference":
        if rank != 0:
            return
        import torch
        from oracle import vsa_oracle as O
        res = run_cpu(cfg, steps=max(1, min(args.steps, 3)), warmup=1)
        be = O.block_elements(cfg["block_size"])
        line = {"metric": "VSA fwd+bwd useful TFLOPS, 92k tok blk64 bf16" if args.workload == DEFAULT_WORKLOAD
                else f"VSA fwd+bwd useful TFLOPS ({args.workload})",
                "value": res["value"], "unit": "TFLOP/s", "n_gpus": args.gpus, "steps": args.steps,
                "warmup": args.warmup, "ms_per_step": res["ms_per_step"], "higher_is_better": True,
                "scaling": "strong", "vs_baseline": None, "dtype": dtype_name(cfg),
                "data": "synthetic N(0,1), seeded", "impl": "reference",
                "config": {"workload": args.workload, "shape_BHLD": [cfg["B"], cfg["H"], cfg["L"], cfg["D"]],
                           "block_elements": be, "topk": cfg["topk"], "gate": cfg["gate"]},
                "cpu_baseline": {k_: res[k_] for k_ in ("value", "unit", "cores", "kind", "sample", "one_thread_value")},
                "e2e": {"value": res["value"], "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
                "gpu_launches": 0}
        print(json.dumps(line), flush=True)
        return

    if args.impl == "reference_triton" and (args.gpus == 1 or world > 1):
        return run_reference_gpu(args, cfg, rank, world, local_rank)
    if args.gpus > 1 and world == 1:
        # launched plainly with --gpus N: re-launch under torchrun, one rank per GPU
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={args.gpus}",
               "--master-addr", "127.0.0.1", "--master-port", os.environ.get("MASTER_PORT", "29533"),
               os.path.abspath(__file__)] + sys.argv[1:]
        sys.exit(subprocess.call(cmd))
    if world != args.gpus:
        print(f"warning: --gpus {args.gpus} but WORLD_SIZE={world}; using WORLD_SIZE", file=sys.stderr)
    run_gpu(args, cfg, rank, world, local_rank)


if __name__ == "__main__":
    main()
