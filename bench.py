#!/usr/bin/env python
"""Benchmark of the fused TriMul forward on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference|nccl_baseline]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

Workload: the README shape of the reference -- z (1, 4096, 4096, 256) bf16 ~ N(0,1), outgoing,
mask of ones, LayerNorm affine off identity, six projection matrices ~ N(0, 1/D), biases 0,
seeded -- sharded over a flat 1-D cp mesh with cp = N GPUs (strong scaling: total work fixed).
Metric: TriMul forward TFLOP/s with FLOPs = 2*B*D*N^3 + 12*B*N^2*D^2.

One JSON line is printed by rank 0.  ``value`` is timed with inputs resident in HBM (CUDA events
on the launching stream, max over ranks); ``e2e`` times the same forward through the public
module with pinned-host input and output copies inside the window; ``roofline`` reports the
dominant kernel (the triangle contraction) against the measured bf16 tensor peak; ``cpu_baseline``
times the CPU oracle (a port of the reference's eager TriMul) on a bounded sample.

``--impl reference`` times the reference's eager PyTorch TriMul on the host cores (the reference's
fused kernels are SM90-only and refuse to run on sm_100), on a bounded sample of the workload.
``--impl nccl_baseline`` runs the conventional context-parallel form (eager PyTorch kernels + NCCL
all-gather / reduce-scatter, ``baseline/nccl_cp_trimul.py``) on the same workload and GPUs.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

REPO = Path(__file__).resolve().parent
sys.path.insert(0, str(REPO))

import torch  # noqa: E402

WORKLOADS = {
    # B, N, D; default direction; token-grid mesh ("1d": rows over all ranks, "2d": (2, ranks/2) rows x columns);
    # pair mask ("ones", or "pad": outer product of a token mask whose last 10 % is zero)
    "readme_n4096_d256": dict(B=1, N=4096, D=256, direction="outgoing", mesh="1d", mask="ones"),
    "mesh2x4_incoming_pad_n4096_d256": dict(B=1, N=4096, D=256, direction="incoming", mesh="2d", mask="pad"),
    "large_n8192_d128": dict(B=2, N=8192, D=128, direction="outgoing", mesh="1d", mask="ones"),
    "single_n1024_d128": dict(B=1, N=1024, D=128, direction="outgoing", mesh="1d", mask="ones"),
    # the wide feature widths the reference pins at cp=1 (N=2048; 32.7 / 43.9 ms on H100)
    "wide_n2048_d384": dict(B=1, N=2048, D=384, direction="outgoing", mesh="1d", mask="ones"),
    "wide_n2048_d512": dict(B=1, N=2048, D=512, direction="outgoing", mesh="1d", mask="ones"),
    "smoke_n256_d128": dict(B=1, N=256, D=128, direction="outgoing", mesh="1d", mask="ones"),
    # small cases for ncu captures (inputs > L2, < 2 GB on the device)
    "profile_n1024_d256": dict(B=1, N=1024, D=256, direction="outgoing", mesh="1d", mask="ones"),
    "profile_n2048_d128": dict(B=1, N=2048, D=128, direction="outgoing", mesh="1d", mask="ones"),
    "profile_n2048_d256": dict(B=1, N=2048, D=256, direction="outgoing", mesh="1d", mask="ones"),
    "profile_n1024_d512": dict(B=1, N=1024, D=512, direction="outgoing", mesh="1d", mask="ones"),
}
CPU_SAMPLE_N = 768  # token extent of the bounded CPU sample (same D, same distributions)
E2E_MAX_BYTES = 24 << 30  # per-rank input size beyond which the pinned-host end-to-end leg is skipped


def workload(args):
    w = dict(WORKLOADS[args.workload])
    if args.direction:
        w["direction"] = args.direction
    return w


def flops(B, N, D):
    return 2.0 * B * D * N ** 3 + 12.0 * B * N * N * D * D


def measured_peaks():
    p = REPO / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return {"bf16_tflops": float(d["bf16_tflops"]), "bf16_tflops_sustained": float(d["bf16_tflops_sustained"]),
                "hbm_gbs": float(d["hbm_gbs"]), "source": "measured"}
    return {"bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "hbm_gbs": 6650.0, "source": "fallback"}


#: DRAM bytes (read + write) the contraction kernel moves per channel plane, from one-pass ncu captures of whole
#: launches (profiles/tri_contract_kernel_n1024_d256.md, profiles/tri_contract_kernel_n4096_d256.md).  Planes are
#: independent, so a launch moves planes x this; it does NOT scale with N^2: first touch only at N=1024 (a plane
#: pair is 4 MB), 2.2x first touch at N=4096 (a plane pair is 64 MB and part of the tile re-reads miss L2).
KB_DRAM_BYTES_PER_PLANE = {1024: 1.6207e9 / 256, 4096: (48.14e9 + 8.58e9) / 256}


class ClockSampler:
    """Samples SM clock and clock-event (throttle) reasons every 10 ms through NVML (read-only) from
    warm-up to the end of the timed work.  The report prefers the samples that fall inside the timed
    steps; when the timed region is too short to hold three samples it widens to everything sampled
    under load (warm-up, timed steps, per-stage passes) and says so in `window`."""

    REASONS = ((0x8, "hw_slowdown"), (0x40, "hw_thermal_slowdown"), (0x20, "sw_thermal_slowdown"), (0x4, "sw_power_cap"))

    def __init__(self, device: torch.device):
        self.device = device
        self.samples = []   # (host time, sm MHz, reason bitmask)
        self.max_mhz = None
        self.t_load = self.t0 = self.t1 = None
        self._stop = threading.Event()
        self._thread = None
        self.error = None

    def _handle(self, nv):
        try:
            pr = torch.cuda.get_device_properties(self.device)
            bus = "%08x:%02x:%02x.0" % (pr.pci_domain_id, pr.pci_bus_id, pr.pci_device_id)
            return nv.nvmlDeviceGetHandleByPciBusId(bus.encode())
        except Exception:
            return nv.nvmlDeviceGetHandleByIndex(self.device.index or 0)

    def start(self):
        try:
            import pynvml as nv
            nv.nvmlInit()
            h = self._handle(nv)
            self.max_mhz = float(nv.nvmlDeviceGetMaxClockInfo(h, nv.NVML_CLOCK_SM))
            reasons_fn = getattr(nv, "nvmlDeviceGetCurrentClocksEventReasons", None) or \
                getattr(nv, "nvmlDeviceGetCurrentClocksThrottleReasons")

            def pump():
                while not self._stop.is_set():
                    try:
                        self.samples.append((time.time(), float(nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM)),
                                             int(reasons_fn(h))))
                    except Exception as e:  # keep what was sampled
                        self.error = repr(e)
                        return
                    self._stop.wait(0.01)

            self._thread = threading.Thread(target=pump, daemon=True)
            self._thread.start()
        except Exception as e:
            self.error = repr(e)
        self.t_load = time.time()
        return self

    def mark_begin(self):
        self.t0 = time.time()

    def mark_end(self):
        self.t1 = time.time()

    def _summary(self, lo, hi):
        sm, bits = [], 0
        for ts, mhz, r in self.samples:
            if lo <= ts <= hi:
                sm.append(mhz)
                bits |= r
        sm.sort()
        out = {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": self.max_mhz,
               "reasons": [name for bit, name in self.REASONS if bits & bit], "samples": len(sm)}
        if self.error:
            out["error"] = self.error
        return out

    def stop(self):
        t_stop = time.time()
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2)
        if self.t0 is not None and self.t1 is not None:
            r = self._summary(self.t0, self.t1)
            if r["samples"] >= 3:
                r["window"] = "timed steps"
                return r
        r = self._summary(self.t_load, t_stop)
        r["window"] = "warm-up + timed steps + per-stage passes (timed region shorter than three 10 ms samples)"
        return r


def make_layer_weights(D, seed, device):
    """Seeded weights of the benchmark configuration: gains 1 + 0.1 N, LN biases 0.1 N, projection
    matrices N(0, 1/D), projection biases absent."""
    g = torch.Generator().manual_seed(seed)
    rn = lambda *s: torch.randn(*s, generator=g)
    w = {
        "norm_in_w": 1 + 0.1 * rn(D), "norm_in_b": 0.1 * rn(D), "norm_out_w": 1 + 0.1 * rn(D), "norm_out_b": 0.1 * rn(D),
        "p_in_w": rn(2 * D, D) / D ** 0.5, "g_in_w": rn(2 * D, D) / D ** 0.5,
        "p_out_w": rn(D, D) / D ** 0.5, "g_out_w": rn(D, D) / D ** 0.5,
        "p_in_b": None, "g_in_b": None, "p_out_b": None, "g_out_b": None,
    }
    return {k: (None if v is None else v.to(device)) for k, v in w.items()}


def _cpu_sample(D, n_sample):
    w = make_layer_weights(D, 0, "cpu")
    x = torch.randn(1, n_sample, n_sample, D, generator=torch.Generator().manual_seed(1))
    m = torch.ones(1, n_sample, n_sample)
    return w, x, m


def cpu_reference_time(D, direction, threads, n_sample=CPU_SAMPLE_N, reps=2):
    """Time the two CPU spellings of the reference's eager fp32 TriMul at a reduced token extent: the
    op-for-op restatement of ``trimul_ref`` and the eager-module form (fused LayerNorm, biases inside the
    GEMMs).  Returns {name: (seconds, TFLOP/s)}."""
    from oracle.trimul_oracle import trimul_eager_module, trimul_oracle

    torch.set_num_threads(threads)
    w, x, m = _cpu_sample(D, n_sample)
    out = {}
    for name, fn in (("trimul_ref", trimul_oracle), ("eager_module", trimul_eager_module)):
        fn(x[:, :64, :64].contiguous(), direction, m[:, :64, :64].contiguous(), **w)  # warm-up
        best = float("inf")
        for _ in range(reps):
            t0 = time.perf_counter()
            fn(x, direction, m, **w)
            best = min(best, time.perf_counter() - t0)
        out[name] = (best, flops(1, n_sample, D) / best / 1e12)
    return out


def run_reference(args):
    """--impl reference: the reference's eager TriMul on the host cores, in the faster of its two
    spellings (the eager nn.Module form), restated in oracle/ and pinned to the reference's outputs."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    wl = workload(args)
    B, N, D = wl["B"], wl["N"], wl["D"]
    cores = os.cpu_count() or 1
    n_sample = CPU_SAMPLE_N
    from oracle.trimul_oracle import trimul_eager_module

    torch.set_num_threads(cores)
    w, x, m = _cpu_sample(D, n_sample)
    for _ in range(max(1, min(args.warmup, 1))):
        trimul_eager_module(x, wl["direction"], m, **w)
    times = []
    for _ in range(args.steps):
        t0 = time.perf_counter()
        trimul_eager_module(x, wl["direction"], m, **w)
        times.append(time.perf_counter() - t0)
    dt = sum(times) / len(times)
    tf = flops(1, n_sample, D) / dt / 1e12
    sample = (f"one forward at N={n_sample} (same D={D}, same distributions) per step, eager-module spelling, "
              f"{flops(1, n_sample, D):.3e} FLOP; the full N={N} workload is {flops(B, N, D):.3e} FLOP")
    line = {
        "impl": "reference", "metric": "trimul_fwd_tflops", "value": tf, "unit": "TFLOP/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": args.workload, "B": B, "N": N, "D": D, "direction": wl["direction"],
                   "note": "reference fused kernels are SM90-only; its eager PyTorch TriMul timed on host cores"},
        "cpu_baseline": {"value": tf, "unit": "TFLOP/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": tf, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def run_nccl_baseline(args):
    """--impl nccl_baseline: eager PyTorch kernels + NCCL collectives (baseline/nccl_cp_trimul.py) on the same
    workload and GPUs: the conventional context-parallel form the fused path is compared with on this box."""
    import torch.distributed as dist

    from baseline.nccl_cp_trimul import NcclCpTriMul

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}; launch with torch.distributed.run")
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    wl = workload(args)
    B, N, D = wl["B"], wl["N"], wl["D"]
    args.direction = wl["direction"]
    n_loc = N // world
    w = make_layer_weights(D, 0, dev)
    gen = torch.Generator(device="cpu").manual_seed(100 + rank)
    x = torch.empty(B, n_loc, N, D, dtype=torch.bfloat16, device=dev)
    chunk = max(1, n_loc // 8)
    for i0 in range(0, n_loc, chunk):
        x[:, i0:i0 + chunk] = torch.randn(B, min(chunk, n_loc - i0), N, D, generator=gen).to(torch.bfloat16).to(dev)
    m = torch.ones(B, n_loc, N, dtype=torch.bfloat16, device=dev)
    mod = NcclCpTriMul(w)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    n_warm = max(3, args.warmup)
    for _ in range(n_warm):
        out = mod.forward(x, args.direction, m)
    del out
    barrier()
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
    ev[0].record()
    for _ in range(args.steps):
        out = mod.forward(x, args.direction, m)
    ev[1].record()
    barrier()
    t = torch.tensor([ev[0].elapsed_time(ev[1]) / args.steps], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item())
    if rank == 0:
        fl = flops(B, N, D)
        print(json.dumps({
            "impl": "nccl_baseline", "metric": "trimul_fwd_tflops", "value": fl / (ms * 1e-3) / 1e12, "unit": "TFLOP/s",
            "n_gpus": world, "steps": args.steps, "warmup": n_warm, "ms_per_step": ms, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": args.workload, "B": B, "N": N, "D": D, "direction": args.direction,
                       "parallelism": f"cp{world}", "note": "eager PyTorch kernels + NCCL all-gather / reduce-scatter"},
            "gpu_launches": 0}), flush=True)
    if world > 1:
        dist.destroy_process_group()


def token_mask(kind, N):
    """(N,) token mask of the workload: all ones, or the last 10 % of the tokens zero (padding)."""
    m = torch.ones(N)
    if kind == "pad":
        m[int(0.9 * N):] = 0.0
    return m


def run_ours(args):
    import torch.distributed as dist
    from torch.distributed.tensor import DTensor, Shard

    from fold_cp_ops_b200.distributed import DistributedManager
    from fold_cp_ops_b200.distributed.trimul_weights import trimul_module_from_weights
    from fold_cp_ops_b200.distributed.workflows.trimul_autotuned import TriangularMultiplication

    world = int(os.environ.get("WORLD_SIZE", "1"))
    if "RANK" not in os.environ:  # plain `python bench.py`: a one-rank env:// launch
        os.environ.update(RANK="0", WORLD_SIZE="1", LOCAL_RANK="0", LOCAL_WORLD_SIZE="1",
                          MASTER_ADDR="127.0.0.1", MASTER_PORT=str(29500 + os.getpid() % 2000))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}; launch with torch.distributed.run")
    wl = workload(args)
    B, N, D, direction = wl["B"], wl["N"], wl["D"], wl["direction"]
    DistributedManager.initialize(device_type="cuda")
    DistributedManager.init_nvshmem()
    dm = DistributedManager()
    rank, cp, dev = dm.rank, dm.world_size, dm.device
    from collections import OrderedDict

    two_d = wl["mesh"] == "2d" and cp >= 4 and cp % 2 == 0
    DistributedManager.create_grid_group(OrderedDict(cp=(2, cp // 2) if two_d else cp))
    mesh = dm.device_mesh_subgroups if two_d else dm.device_mesh
    placements = [Shard(1), Shard(2)] if two_d else [Shard(1)]
    cp0, cp1 = (2, cp // 2) if two_d else (cp, 1)
    coord = mesh.get_coordinate() if cp > 1 else [0, 0]
    r0, r1 = (coord[0], coord[1]) if two_d else (rank, 0)
    ni, nj = N // cp0, N // cp1
    i_off, j_off = r0 * ni, r1 * nj
    torch.manual_seed(0)
    w = make_layer_weights(D, 0, dev)
    layer = trimul_module_from_weights(w)
    tuning = None
    if args.contract_form is not None or args.contract_band is not None or args.contract_fixed_start or args.contract_pace is not None:
        from fold_cp_ops_b200.distributed.workflows.trimul_tuning import BackTuning, TriMulTuning

        tuning = TriMulTuning(back=BackTuning(contract_form=args.contract_form, band_rows=args.contract_band,
                                                  fixed_start=True if args.contract_fixed_start else None,
                                                  pace_ns=args.contract_pace))
    trimul = TriangularMultiplication(layer, direction, mesh if cp > 1 else None, dm, placements=placements if cp > 1 else None,
                                      dtype=torch.bfloat16, tuning=tuning)
    gen = torch.Generator(device="cpu").manual_seed(100 + rank)
    x_bytes = B * ni * nj * D * 2
    do_e2e = not args.kernels_only and not args.no_e2e and x_bytes <= E2E_MAX_BYTES
    # the local block is generated in slices (a full fp32 randn of it would not fit comfortably) into
    # pinned host memory -- the end-to-end leg moves it every step -- or straight onto the device
    chunk = max(1, ni // 16)
    if do_e2e:
        x_host = torch.empty(B, ni, nj, D, dtype=torch.bfloat16).pin_memory()
        out_host = torch.empty(B, ni, nj, D, dtype=torch.bfloat16).pin_memory()
        x_dev = None
    else:
        x_host = out_host = None
        x_dev = torch.empty(B, ni, nj, D, dtype=torch.bfloat16, device=dev)
    for b in range(B):
        for i0 in range(0, ni, chunk):
            piece = torch.randn(min(chunk, ni - i0), nj, D, generator=gen).to(torch.bfloat16)
            (x_host if do_e2e else x_dev)[b, i0:i0 + chunk] = piece
    tm = token_mask(wl["mask"], N)
    m_local = (tm[i_off:i_off + ni, None] * tm[None, j_off:j_off + nj]).to(torch.bfloat16).expand(B, ni, nj).contiguous()
    m_host = m_local.pin_memory() if do_e2e else None
    if do_e2e:
        x_dev = x_host.to(dev, non_blocking=True)
    m_dev = m_local.to(dev)

    def wrap(t, gshape):
        if cp == 1:
            return t
        st = torch.empty(gshape, device="meta").stride()
        return DTensor.from_local(t, mesh, placements, shape=torch.Size(gshape), stride=st, run_check=False)

    x_in, m_in = wrap(x_dev, (B, N, N, D)), wrap(m_dev, (B, N, N))
    trimul.prepare(n_token=N, batch=B, masked=True)

    def barrier():
        if cp > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def step_resident():
        return trimul(x_in, m_in)

    def step_e2e():
        xd = x_host.to(dev, non_blocking=True)
        md = m_host.to(dev, non_blocking=True)
        o = trimul(wrap(xd, (B, N, N, D)), wrap(md, (B, N, N)))
        ol = o.to_local() if cp > 1 else o
        out_host.copy_(ol, non_blocking=True)

    n_warm = args.warmup if args.kernels_only else max(3, args.warmup)
    sampler = ClockSampler(dev).start() if rank == 0 else None
    out = None
    for _ in range(n_warm):
        out = None  # the previous output goes back to the allocator before the next one is made
        out = step_resident()
    barrier()
    # ---- value: inputs resident in HBM ---------------------------------------------------------
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
    barrier()
    if sampler:
        sampler.mark_begin()
    ev[0].record()
    for _ in range(args.steps):
        out = None
        out = step_resident()
    ev[1].record()
    barrier()
    if sampler:
        sampler.mark_end()
    ms = ev[0].elapsed_time(ev[1]) / args.steps
    # ---- per-kernel times and the device timeline (live, on the launching stream) ---------------
    stage_ms = None
    wait_ms = {}
    engines = trimul._live_engines()
    eng = engines[-1] if engines else None
    if eng is not None and (args.stage_times or not args.kernels_only):
        # kernel-only CUDA-event windows (the flag kernels are outside them) and, at cp > 1, the time each
        # rank's stream sat in the three cross-rank flag waits (from %globaltimer stamps in the wait kernels)
        trimul.collect_stats(True)
        runs = []
        for _ in range(3):
            out = None
            out = step_resident()
            runs.append(trimul.last_forward_stats())
        trimul.collect_stats(False)
        med = lambda vals: sorted(vals)[len(vals) // 2]
        stage_ms = {k: med([r["stage_ms"][k] for r in runs]) for k in runs[0]["stage_ms"]}
        wait_ms = {k: med([r["wait_ms"].get(k) or 0.0 for r in runs]) for k in runs[0]["wait_ms"]}
    clocks = sampler.stop() if sampler else None
    # ---- e2e: pinned host -> device, forward, device -> pinned host, every step -----------------
    # Serial form first (copy in, forward, copy out on one stream: the latency of one request), then the
    # form a throughput-minded caller uses: the same three operations of every step on three streams with
    # double-buffered device inputs, so that the copy-in of step i+1 and the copy-out of step i-1 overlap
    # the forward of step i (PCIe is full duplex).  Every step still moves all of its input and output.
    ms_e2e = ms_e2e_serial = float("nan")
    if do_e2e:
        step_e2e()
        barrier()
        n_serial = min(2, args.steps)
        ev2 = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
        ev2[0].record()
        for _ in range(n_serial):
            step_e2e()
        ev2[1].record()
        barrier()
        ms_e2e_serial = ev2[0].elapsed_time(ev2[1]) / n_serial

        main = torch.cuda.current_stream()
        s_in, s_fw, s_out = (torch.cuda.Stream(device=dev) for _ in range(3))
        xd = [torch.empty_like(x_dev) for _ in range(2)]
        md = [torch.empty_like(m_dev) for _ in range(2)]
        in_ready = [torch.cuda.Event() for _ in range(2)]
        fw_done = [torch.cuda.Event() for _ in range(2)]
        for st in (s_in, s_fw, s_out):
            st.wait_stream(main)

        def step_pipelined(i):
            b = i & 1
            with torch.cuda.stream(s_in):
                s_in.wait_event(fw_done[b])          # the forward that read this input buffer has finished
                xd[b].copy_(x_host, non_blocking=True)
                md[b].copy_(m_host, non_blocking=True)
                in_ready[b].record(s_in)
            with torch.cuda.stream(s_fw):
                s_fw.wait_event(in_ready[b])
                o = trimul(wrap(xd[b], (B, N, N, D)), wrap(md[b], (B, N, N)))
                ol = o.to_local() if cp > 1 else o
                fw_done[b].record(s_fw)
            with torch.cuda.stream(s_out):
                s_out.wait_event(fw_done[b])
                ol.record_stream(s_out)
                out_host.copy_(ol, non_blocking=True)

        def drain():
            for st in (s_in, s_fw, s_out):
                main.wait_stream(st)
            barrier()

        step_pipelined(0)
        step_pipelined(1)
        drain()
        ev3 = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
        for st in (s_in, s_fw, s_out):
            st.wait_stream(main)
        ev3[0].record(main)
        for st in (s_in, s_fw, s_out):
            st.wait_stream(main)
        n_pipe = max(args.steps, 4)
        for i in range(n_pipe):
            step_pipelined(i)
        for st in (s_in, s_fw, s_out):
            main.wait_stream(st)
        ev3[1].record(main)
        barrier()
        ms_e2e = ev3[0].elapsed_time(ev3[1]) / n_pipe
        del xd, md
    # ---- reduce over ranks (max) ----------------------------------------------------------------
    order = ("ln_gated_proj", "tri_contract", "ln_out_proj")
    waits = ("front", "back", "consumed")
    vals = [ms, ms_e2e, ms_e2e_serial] + ([stage_ms[k] for k in order] if stage_ms else [0, 0, 0]) + \
        [wait_ms.get(k, 0.0) for k in waits] + [sum(wait_ms.get(k, 0.0) for k in waits)]
    t = torch.tensor(vals, device=dev, dtype=torch.float64)
    tmin = t.clone()
    if cp > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dist.all_reduce(tmin, op=dist.ReduceOp.MIN)
    ms, ms_e2e, ms_e2e_serial, t_a, t_b, t_c, w_front, w_back, w_cons, w_total = t.tolist()
    w_min = tmin.tolist()[6:9]
    w_total_min = tmin.tolist()[9]
    trimul.check()  # raises if any bounded device-side wait of the run expired
    # ---- parity spot check at full size: every rank checks a patch of its own block against the oracle ----
    verify = None
    if args.verify and not args.kernels_only:
        verify = spot_check(w, x_dev, out.to_local() if cp > 1 else out, wl, direction, cp, cp0, cp1, rank, r0, r1, dev)
    if rank == 0:
        peaks = measured_peaks()
        fl = flops(B, N, D)
        tf = fl / (ms * 1e-3) / 1e12
        # dominant kernel: the contraction.  One launch contracts planes_b batch planes of this rank's D/cp
        # channels (planes_b = B unless the workspace was capped to one batch plane per launch); the stage
        # windows time ONE launch, so the algorithmic FLOPs beside them are those of one launch
        planes_b = getattr(next(iter(eng._ws.values())), "planes_b", B) if eng is not None and eng._ws else B
        planes_per_launch = planes_b * (D // cp)
        fl_b = 2.0 * planes_per_launch * N ** 3
        ach = fl_b / (t_b * 1e-3) / 1e12 if t_b > 0 else None
        peak = peaks["bf16_tflops_sustained"]
        roof = {"bound": "tensor", "kernel": "tri_contract_pair_kernel", "achieved": ach, "peak": peak, "unit": "TFLOP/s",
                "frac": (ach / peak) if ach else None,
                "traffic": (KB_DRAM_BYTES_PER_PLANE[N] * planes_per_launch) if N in KB_DRAM_BYTES_PER_PLANE else None,
                "traffic_unit": "DRAM bytes per launch: one-pass ncu capture of a whole launch at this N, times the "
                                "planes of one launch / the captured 256 (planes are independent); null where this N "
                                "was not captured",
                "traffic_first_touch": 6.0 * planes_per_launch * N * N,
                "peak_source": f"{peaks['source']} (sustained: the kernel runs inside a long step)",
                "frac_of_burst_peak": (ach / peaks["bf16_tflops"]) if ach else None,
                "stage_ms": {"ln_gated_proj": t_a, "tri_contract": t_b, "ln_out_proj": t_c},
                "stage_ms_note": "CUDA events around each kernel alone (max over ranks); the flag kernels between "
                                 "them are outside these windows",
                "launches_per_kernel_per_step": B // planes_b}
        # whole-step roofline: the slowest of tensor time, HBM time (9 S per rank) and NVLink egress (3 S (cp-1)/cp)
        S = B * N * N * D * 2.0 / cp
        t_tc = fl / cp / (peaks["bf16_tflops_sustained"] * 1e12) * 1e3
        t_hbm = 9.0 * S / (peaks["hbm_gbs"] * 1e9) * 1e3
        t_nvl = 3.0 * S * (cp - 1) / cp / 770e9 * 1e3
        roof["step"] = {"roof_ms": max(t_tc, t_hbm, t_nvl), "tensor_ms": t_tc, "hbm_ms": t_hbm, "nvlink_ms": t_nvl,
                        "frac": max(t_tc, t_hbm, t_nvl) / ms,
                        "frac_of_burst_tensor_peak": fl / cp / (peaks["bf16_tflops"] * 1e12) * 1e3 / ms,
                        "note": "tensor term against the measured sustained bf16 rate, HBM against the measured copy "
                                "rate, NVLink against the measured 770 GB/s peer copy per direction"}
        if cp > 1 and t_a > 0 and t_b > 0:
            # the reshards ride the two store epilogues: bytes this rank sends to peers / kernel time
            roof["nvlink_gbs"] = {"front_in_ln_gated_proj": 2.0 * S * (cp - 1) / cp / (t_a * 1e-3) / 1e9,
                                  "back_in_tri_contract": S * (cp - 1) / cp / (t_b * 1e-3) / 1e9,
                                  "wait_ms_max_over_ranks": {"front": w_front, "back": w_back, "consumed": w_cons},
                                  "wait_ms_min_over_ranks": dict(zip(waits, w_min)),
                                  "exposed_ms": w_total, "exposed_ms_min_over_ranks": w_total_min,
                                  "note": "egress per rank = algorithmic bytes / kernel-only window; exposed = the largest "
                                          "per-rank total of time spent inside the three cross-rank flag waits of one "
                                          "forward, measured on the device (%globaltimer at wait entry and exit): reshard "
                                          "time that was not hidden behind a kernel, rank skew included"}
        cpu = None
        if not args.kernels_only and cp == 1:  # the CPU baseline is reported on rank 0 of the one-GPU run only
            cores = os.cpu_count() or 1
            both = cpu_reference_time(D, direction, cores)
            name = max(both, key=lambda k: both[k][1])
            cpu = {"value": both[name][1], "unit": "TFLOP/s", "cores": cores, "kind": "port",
                   "sample": f"{name} spelling of the reference's eager forward at N={CPU_SAMPLE_N}, D={D} (best of 2, "
                             f"{both[name][0]:.2f} s each); FLOPs scale as 2*D*N^3 + 12*N^2*D^2",
                   "spellings_tflops": {k: v[1] for k, v in both.items()}}
        bytes_in = B * ni * nj * D * 2 + B * ni * nj * 2
        bytes_out = B * ni * nj * D * 2
        e2e = None
        if do_e2e:
            e2e = {"value": fl / (ms_e2e * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": ms_e2e,
                   "h2d_bytes_per_step": bytes_in, "d2h_bytes_per_step": bytes_out,
                   "mode": "every step copies its input from pinned host memory and its output back; copy-in, "
                           "forward and copy-out of consecutive steps overlap on three streams",
                   "serial_ms_per_step": ms_e2e_serial,
                   "serial_value": fl / (ms_e2e_serial * 1e-3) / 1e12}
        n_kernels = 3 * (B // max(1, getattr(next(iter(eng._ws.values())), "planes_b", B))) if eng is not None and eng._ws else 3
        line = {
            "metric": "trimul_fwd_tflops", "value": tf, "unit": "TFLOP/s", "n_gpus": cp, "steps": args.steps,
            "warmup": n_warm, "ms_per_step": ms, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": args.workload, "B": B, "N": N, "D": D, "direction": direction,
                       "parallelism": f"cp{cp}" if not two_d else f"cp{cp0}x{cp1}",
                       "mesh": "2-D, rows x columns sharded" if two_d else "1-D, rows sharded", "mask": wl["mask"],
                       "l2": "inputs (>= 1 GB per rank) exceed the 126 MB L2; no flush needed",
                       "contract_form": args.contract_form or "engine default",
                       "contract_band_rows": args.contract_band if args.contract_band is not None else "engine default",
                       "contract_fixed_start": bool(args.contract_fixed_start),
                       "contract_pace_ns": args.contract_pace if args.contract_pace is not None else "engine default"},
            "clocks": clocks,
            "e2e": e2e if e2e is not None else {"value": None, "unit": "TFLOP/s", "h2d_bytes_per_step": bytes_in,
                                                "d2h_bytes_per_step": bytes_out,
                                                "skipped": "not run for this invocation (--kernels-only / --no-e2e, or "
                                                           "the per-rank input exceeds the pinned-host budget)"},
            "gpu_launches": args.steps * (n_kernels if cp == 1 else n_kernels + 6),
            "roofline": roof, "cpu_baseline": cpu,
        }
        if verify is not None:
            line["verify"] = verify
        print(json.dumps(line), flush=True)
    trimul.free()
    DistributedManager.cleanup()


def spot_check(w, x_local, out_local, wl, direction, cp, cp0, cp1, rank, r0, r1, dev, rows=2, cols=64):
    """Every rank compares a (rows x cols) patch of ITS OWN output block with the fp32 oracle evaluated
    from the GLOBAL input.  The input lines the patch needs (whole rows of x for "outgoing", whole columns
    for "incoming") live on other ranks: every rank publishes which lines it needs, everybody fills the
    parts it owns into one zero tensor, and a sum over the ranks assembles them (exact: one non-zero
    term per element).  The columns of the patch are chosen next to an owner boundary, so the lines
    come from at least two different ranks.  Runs outside every timed region."""
    import torch.distributed as dist

    from oracle.trimul_oracle import layer_norm

    B, N, D = wl["B"], wl["N"], wl["D"]
    ni, nj = N // cp0, N // cp1
    i_off, j_off = r0 * ni, r1 * nj
    b = B - 1
    n_line = rows + cols
    # output patch: rows ii and columns jj of this rank's block (global indices)
    ii = i_off + (torch.arange(rows) * 7 + 3) % ni
    # the lines of the jj side are indexed along the OTHER token axis: put them across a boundary of the
    # blocks that axis is split into (rows are split cp0 ways), staying inside this rank's column block
    line_block = N // cp0
    edge = ((j_off // line_block) + 1) * line_block      # first boundary at or after the block's start
    if not (j_off < edge < j_off + nj and cp0 > 1):
        edge = j_off + nj // 2
    jj = torch.arange(edge - cols // 2, edge + cols // 2).clamp_(j_off, j_off + nj - 1)
    need = torch.cat([ii, jj]).to(dev)
    if cp > 1:
        all_need = torch.empty(cp * n_line, dtype=need.dtype, device=dev)
        dist.all_gather_into_tensor(all_need, need)
    else:
        all_need = need
    lines = torch.zeros(all_need.numel(), N, D, dtype=torch.bfloat16, device=dev)
    want = all_need.tolist()
    for idx, g in enumerate(want):
        if direction == "outgoing":       # line g = x[b, g, :, :]; this rank owns columns [j_off, j_off + nj) of rows in its block
            if i_off <= g < i_off + ni:
                lines[idx, j_off:j_off + nj] = x_local[b, g - i_off]
        else:                             # line g = x[b, :, g, :]
            if j_off <= g < j_off + nj:
                lines[idx, i_off:i_off + ni] = x_local[b, :, g - j_off]
    if cp > 1:
        dist.all_reduce(lines)
    mine = lines[rank * n_line:(rank + 1) * n_line].float()
    del lines
    torch.backends.cuda.matmul.allow_tf32 = False
    wf = {k: (None if v is None else v.float()) for k, v in w.items()}
    tm = token_mask(wl["mask"], N).to(dev)
    xn = layer_norm(mine, wf["norm_in_w"], wf["norm_in_b"], 1e-5)                  # (lines, N, D)
    ab = (xn @ wf["p_in_w"].T) * torch.sigmoid(xn @ wf["g_in_w"].T)
    ab = ab * (tm[need.long()][:, None] * tm[None, :])[..., None]                    # pair mask = outer product
    a, bb = ab[:rows, :, :D], ab[rows:, :, D:]
    tri = torch.einsum("ikd,jkd->ijd", a, bb)
    trin = layer_norm(tri, wf["norm_out_w"], wf["norm_out_b"], 1e-5)
    x_ij = x_local[b][(ii - i_off).to(dev)][:, (jj - j_off).to(dev)].float()
    ref = (trin @ wf["p_out_w"].T) * torch.sigmoid(layer_norm(x_ij, wf["norm_in_w"], wf["norm_in_b"], 1e-5) @ wf["g_out_w"].T)
    got = out_local[b][(ii - i_off).to(dev)][:, (jj - j_off).to(dev)].float()
    err = (got - ref).abs()
    ok = bool((err <= 2e-2 + 6e-2 * ref.abs()).all().item())
    stats = torch.tensor([err.max().item(), (err / ref.abs().clamp_min(1e-2)).max().item(), 0.0 if ok else 1.0,
                          float(ref.abs().max().item())], device=dev, dtype=torch.float64)
    if cp > 1:
        dist.all_reduce(stats, op=dist.ReduceOp.MAX)
    mx, rel, bad, refmax = stats.tolist()
    return {"ranks_checked": cp, "patch_per_rank": [rows, cols], "batch_index": b, "max_abs_err": mx, "max_rel_err": rel,
            "max_abs_ref": refmax, "bound": "|err| <= 2e-2 + 6e-2*|ref| per element (the reference's distributed gate)",
            "within_bound_on_every_rank": bad == 0.0,
            "lines": "input lines gathered from their owner ranks; patch columns straddle an owner boundary"}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", choices=("ours", "reference", "nccl_baseline"), default="ours")
    ap.add_argument("--workload", choices=sorted(WORKLOADS), default="readme_n4096_d256")
    ap.add_argument("--direction", choices=("outgoing", "incoming"), default=None,
                    help="override the workload's own direction")
    ap.add_argument("--kernels-only", action="store_true",
                    help="time the resident-input forward only (skip the e2e, CPU-baseline and verify legs); for profilers")
    ap.add_argument("--no-e2e", action="store_true", help="skip the pinned-host end-to-end leg")
    ap.add_argument("--contract-pace", type=int, default=None,
                    help="longest wait (ns) of a CTA pair of the contraction for the other pairs before a tile; "
                         "0 = the library's choice, negative = off")
    ap.add_argument("--contract-fixed-start", action="store_true",
                    help="every rank walks the contraction's tiles from tile (0, 0) instead of from its own block")
    ap.add_argument("--contract-band", type=int, default=None,
                    help="tile rows per band of the contraction kernel's tile walk (1 = row-major; default: the engine's choice)")
    ap.add_argument("--contract-form", choices=("pair", "single"), default=None,
                    help="force the contraction kernel's form (default: the engine's choice, CTA pairs when the shape allows)")
    ap.add_argument("--stage-times", action="store_true",
                    help="with --kernels-only: still report the per-kernel times (used with profiling builds of the "
                         "library selected by CPO_TRIMUL_LIB, whose results are wrong by construction)")
    ap.add_argument("--verify", action="store_true", default=True)
    ap.add_argument("--no-verify", dest="verify", action="store_false")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    elif args.impl == "nccl_baseline":
        run_nccl_baseline(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
