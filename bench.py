#!/usr/bin/env python
"""Benchmark of the PoM layer hot path (forward + backward) on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload dit|masked|seq64k|seq64k_causal]
    python bench.py --impl reference ...        # CPU restatement of the reference path, same metric

One "step" is one forward + backward pass of one PoM layer over one batch of seeded synthetic
input, with gradients for the input and all four parameters.  Rank 0 prints one JSON line.

Workloads
  dit            B=32, N=1024 (32x32 patches), D=1152, degree 2, expand 2, bf16, no mask.  With
                 --gpus N every rank runs its own batch of 32 samples (weak scaling, no collective
                 on the data path: samples are independent).
  dit_heads16    dit with n_sel_heads=16 (one gate value per head, as the reference's own benchmarks instantiate the
                 layer): the query side collapses to (heads x D) matrices per sample, see csrc/pom_heads.cu.
  masked         B=64, N=2048, D=1024, degree 3, expand 2, key-padding mask (lengths U[256, 2048]).
  seq64k         B=1, N=65536 (256x256 grid, 2-D rotary), D=1152, token-sharded over the ranks
                 (strong scaling; all-reduce of the (B, P) partial sums, weight-gradient all-reduce
                 inside the timed region).
  seq64k_causal  same, token-causal (all-gather of rank totals + local exclusive scan).
  video          forward only: B=8, 16 frames x 256 tokens, D=1024, degree 2, expand 4, 12 layers of
                 x += PoM.state_forward(x); x += W2 gelu(W1 x), state carried across frames; one step = all 16
                 frames through all layers, replayed as one CUDA graph (metric: tokens/s through the stack).
  video_block    the same stack and result, all 16 frames in one pass: every mixer runs with
                 BlockCausal(256) (per-frame means + running mean over frames), so each GEMM sees 32768 rows.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

WORKLOADS = {
    "dit": dict(B=32, N=1024, D=1152, degree=2, expand=2, mask="none", rope=None, shard="batch"),
    "dit_heads16": dict(B=32, N=1024, D=1152, degree=2, expand=2, mask="none", rope=None, shard="batch", heads=16),
    "masked": dict(B=64, N=2048, D=1024, degree=3, expand=2, mask="keypad", rope=None, shard="batch"),
    "seq64k": dict(B=1, N=65536, D=1152, degree=2, expand=2, mask="none", rope="2d", shard="token"),
    "seq64k_causal": dict(B=1, N=65536, D=1152, degree=2, expand=2, mask="causal", rope="2d", shard="token"),
    "video": dict(B=8, N=4096, D=1024, degree=2, expand=4, mask="block-causal", rope=None, shard="batch",
                  frame=256, layers=12),
    "video_block": dict(B=8, N=4096, D=1024, degree=2, expand=4, mask="block-causal", rope=None, shard="batch",
                        frame=256, layers=12, single_pass=True),
}
METRIC = "pom_layer_fwd_bwd_tokens_per_s"
UNIT = "tokens/s"

# DRAM bytes (read + write) per launch, from the ncu captures summarised under profiles/
# (dram__bytes_read.sum + dram__bytes_write.sum of one launch); None where no capture exists.
NCU_TRAFFIC_BYTES = {
    "gemm[32768x1152x4608 B^T]": 399.2e6,   # profiles/gemm_pair_store_dx_32768x1152x4608.md (algorithmic 388.6e6)
    "ctx_gemm": 189.3e6,                    # profiles/ctx_gemm_dit.md (algorithmic 231.8e6, part still in L2)
}


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        d = json.load(open(path))
        return dict(hbm=d["hbm_gbs"], burst=d["bf16_tflops"], sustained=d.get("bf16_tflops_sustained", d["bf16_tflops"]),
                    source="measured")
    return dict(hbm=6650.0, burst=1590.0, sustained=1400.0, source="fallback")


class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi while the timed region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "50"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._pump, daemon=True).start()
        except OSError:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            if len(r) < 7:
                continue
            try:
                sm.append(float(r[0]))
                mx.append(float(r[1]))
            except ValueError:
                continue
            for n, v in zip(names, r[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def flops_per_step(w, valid_frac=1.0):
    """Algorithmic tensor work of one fwd+bwd step: 18 * M * D * P (projections 4+2 forward, 12 backward)."""
    M, D = w["B"] * w["N"], w["D"]
    P = w["expand"] * D
    if "layers" in w:  # forward only: projections 6 M D P plus the 4 D feed-forward 16 M D^2, per layer
        return w["layers"] * M * (6.0 * D * P + 16.0 * D * D)
    if w.get("heads", 1) > 1:
        # one gate value per head and one aggregate per sample: the query side is (heads x D)-sized, what remains
        # is the (P + heads)-wide input projection forward (2) and its two backward products (2 + 2)
        return 6.0 * M * D * (P + w["heads"])
    return 18.0 * M * D * P


# ------------------------------------------------------------------------------------------- reference arm
def cpu_reference_tokens_per_s(w, steps, warmup, sample_tokens=4096):
    """Times the CPU restatement of the reference path (oracle/pom_oracle.py, fp32, all host threads) on a
    bounded sample of the workload: the same layer and distributions with the batch (or, for one long
    sequence, the token count) cut down so that a step takes about a second."""
    from oracle import pom_oracle as O

    torch.set_num_threads(os.cpu_count() or 1)
    D, K, E = w["D"], w["degree"], w["expand"]
    if "layers" in w:
        return cpu_reference_video(w, steps, warmup, O)
    if w["B"] > 1:
        N = w["N"]
        B = max(1, sample_tokens // N)
    else:
        B, N = 1, sample_tokens
    heads = w.get("heads", 1)
    params = {k: v.requires_grad_(True) for k, v in O.init_params(D, K, E, heads, seed=0).items()}
    rope = None
    kw = {}
    if w["rope"] == "2d":
        side = int(N ** 0.5)
        N = side * side
        rope = O.RopeConfig(two_d=True, max_h=side, max_w=side)
        kw["positions_hw"] = torch.stack([torch.arange(N) // side, torch.arange(N) % side], 1)
    model = O.OraclePoM(params, K, E, heads, rope)
    g = torch.Generator().manual_seed(0)
    x = torch.randn(B, N, D, generator=g).requires_grad_(True)
    gy = torch.randn(B, N, D, generator=g)
    if w["mask"] == "keypad":
        L = torch.randint(256, N + 1, (B,), generator=g)
        kw["mask"] = (torch.arange(N).view(1, N) < L.view(B, 1)).float()
    elif w["mask"] == "causal":
        kw["mask"] = "causal"

    def step():
        y = model.forward(x, **kw)
        torch.autograd.grad(y, [x] + model.parameters(), gy)

    for _ in range(warmup):
        step()
    times = []
    for _ in range(steps):
        t0 = time.perf_counter()
        step()
        times.append(time.perf_counter() - t0)
    sec = statistics.median(times)
    return (B * N) / sec, sec, f"B={B}, N={N} of the workload (fp32, {torch.get_num_threads()} threads), median of {steps}"


def cpu_reference_video(w, steps, warmup, O):
    """Frame loop of the oracle (state_forward + GELU feed-forward) for ONE sample and TWO layers; the
    tokens/s of the full 12-layer stack is the measured figure divided by layers / 2."""
    D, K, E, L = w["D"], w["degree"], w["expand"], w["frame"]
    sample_layers = 2
    g = torch.Generator().manual_seed(0)
    layers = []
    for i in range(sample_layers):
        p = O.init_params(D, K, E, seed=i)
        w1 = (torch.rand(4 * D, D, generator=g) * 2 - 1) / D ** 0.5
        w2 = (torch.rand(D, 4 * D, generator=g) * 2 - 1) / (4 * D) ** 0.5
        layers.append((O.OraclePoM(p, K, E), w1, w2))
    x = torch.randn(1, w["N"], D, generator=g)

    def step():
        states = [None] * sample_layers
        with torch.no_grad():
            for f in range(w["N"] // L):
                h = x[:, f * L:(f + 1) * L]
                for i, (m, w1, w2) in enumerate(layers):
                    y, states[i] = m.state_forward(h, None, states[i])
                    h = h + y
                    h = h + torch.nn.functional.gelu(h @ w1.t()) @ w2.t()

    for _ in range(warmup):
        step()
    times = []
    for _ in range(steps):
        t0 = time.perf_counter()
        step()
        times.append(time.perf_counter() - t0)
    sec = statistics.median(times) * (w["layers"] / sample_layers)
    return w["N"] / sec, sec, (f"B=1, {sample_layers} of {w['layers']} layers timed and scaled by {w['layers'] // sample_layers} "
                               f"(fp32, {torch.get_num_threads()} threads), median of {steps}")


def run_reference(args, w, rank):
    if rank != 0:
        return
    steps = max(1, min(args.steps, 5))
    val, sec, sample = cpu_reference_tokens_per_s(w, steps, min(args.warmup, 1))
    line = {
        "impl": "reference", "metric": METRIC, "value": val, "unit": UNIT, "n_gpus": args.gpus, "steps": steps,
        "warmup": min(args.warmup, 1), "ms_per_step": sec * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": args.workload, **{k: w[k] for k in ("B", "N", "D", "degree", "expand", "mask")}},
        "cpu_baseline": {"value": val, "unit": UNIT, "cores": torch.get_num_threads(), "kind": "port", "sample": sample},
        "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------- B200 arm
def build_case(w, rank, world, device, exchange="nccl"):
    """Module, rotating input sets and call kwargs for this rank."""
    from pom_b200 import PoM, PoMRoPE, SeqShard

    D, K, E = w["D"], w["degree"], w["expand"]
    torch.manual_seed(0)
    if "layers" in w:
        from pom_b200.stack import PoMStack

        mod = PoMStack(D, K, E, w["layers"]).to(device)
        for p in mod.parameters():
            p.data = p.data.to(torch.bfloat16)
        gen = torch.Generator().manual_seed(1000 + rank)
        host_sets = [(torch.randn(w["B"], w["N"], D, generator=gen).to(torch.bfloat16).pin_memory(), None)
                     for _ in range(3)]
        return mod, host_sets, {}, w["B"] * w["N"]
    if w["rope"] == "2d":
        side = int(w["N"] ** 0.5)
        mod = PoMRoPE(D, K, E, 1, 1, rope_2d=True, max_h=side, max_w=side)
    else:
        mod = PoM(D, K, E, 1, w.get("heads", 1))
    mod = mod.to(device)
    for p in mod.parameters():
        p.data = p.data.to(torch.bfloat16)
    B, N = w["B"], w["N"]
    kw = {}
    if w["shard"] == "token":
        n_loc = N // world
        off = rank * n_loc
        if w["rope"] == "2d":
            idx = torch.arange(off, off + n_loc)
            kw["positions_hw"] = torch.stack([idx // side, idx % side], 1).to(device)
        if world > 1:
            peer = None
            if exchange == "peer":
                from pom_b200.peer import PeerExchange

                # collective: either every rank maps its peers or (agreed through a reduction) none uses them
                try:
                    peer = PeerExchange(slot_floats=max(4096, B * D * E),
                                        flat_floats=sum(p.numel() for p in mod.parameters()) + 4)
                    ok = torch.ones(1, device=device)
                except Exception as e:  # e.g. CUDA IPC not permitted between these processes
                    print(f"[bench] peer exchange unavailable on rank {rank}: {e}; using NCCL", file=sys.stderr)
                    ok = torch.zeros(1, device=device)
                torch.distributed.all_reduce(ok, op=torch.distributed.ReduceOp.MIN)
                if float(ok.item()) == 0.0:
                    peer = None
            kw["shard"] = SeqShard(token_offset=off, n_global=N, peer=peer)
        tokens_local = B * n_loc
    else:
        n_loc = N
        tokens_local = B * N
    if w["mask"] == "causal":
        kw["mask"] = "causal"
    gen = torch.Generator().manual_seed(1000 + rank)
    n_sets = 3
    host_sets = []
    for _ in range(n_sets):
        x = torch.randn(B, n_loc, D, generator=gen).to(torch.bfloat16).pin_memory()
        gy = torch.randn(B, n_loc, D, generator=gen).to(torch.bfloat16).pin_memory()
        host_sets.append((x, gy))
    if w["mask"] == "keypad":
        L = torch.randint(256, N + 1, (B,), generator=gen)
        kw["mask"] = (torch.arange(N).view(1, N) < L.view(B, 1)).float().to(device)
    return mod, host_sets, kw, tokens_local


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default="dit", choices=sorted(WORKLOADS))
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--graph", default="off", choices=["on", "off"],
                    help="replay the whole fwd+bwd step as a CUDA graph instead of launching it from Python")
    ap.add_argument("--defer-weight-grad-reduce", action="store_true",
                    help="token-sharded runs: leave the parameter-gradient all-reduce to the caller (as a data-parallel "
                         "optimizer step would do) instead of doing it inside the layer")
    ap.add_argument("--exchange", default="peer", choices=["nccl", "peer"],
                    help="token-sharded runs: carry the cross-rank sums by NCCL calls between kernels, or by the "
                         "library's own peer-memory kernels (graph-capturable; turns --graph on unless given)")
    ap.add_argument("--no-overlap-grad-reduce", action="store_true",
                    help="peer exchange: run the parameter-gradient all-reduce on the main stream after the last GEMM "
                         "instead of on a side stream beside the data-gradient GEMM")
    ap.add_argument("--tokens", type=int, default=0, help="override the workload's tokens per sample (N)")
    args = ap.parse_args()
    w = dict(WORKLOADS[args.workload])
    if args.tokens:
        w["N"] = args.tokens
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))

    if args.impl == "reference":
        run_reference(args, w, rank)
        return

    if os.environ.get("NCCL_DEBUG", "").upper() == "VERSION":
        os.environ["NCCL_DEBUG"] = "WARN"  # keep stdout to the one JSON line
    import torch.distributed as dist
    from pom_b200 import _abi, ops

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the B200 arm has no CPU path (use --impl reference for the CPU arm)")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if _abi.lib().pom_device_check() != 0:
        raise SystemExit("the kernels are built for sm_100a and need a B200-class GPU")
    if world > 1:
        from datetime import timedelta

        # a short timeout turns a mismatched collective into an error instead of a ten-minute stall.
        # NCCL may print a version banner on stdout while the communicator comes up: point fd 1 at stderr
        # for that moment so that stdout carries nothing but the JSON line.
        sys.stdout.flush()
        saved_fd = os.dup(1)
        os.dup2(2, 1)
        try:
            dist.init_process_group("nccl", device_id=device, timeout=timedelta(seconds=180))
            warm = torch.zeros(1, device=device)
            dist.all_reduce(warm)
            torch.cuda.synchronize()
        finally:
            os.dup2(saved_fd, 1)
            os.close(saved_fd)
    args.warmup = max(args.warmup, 3)

    mod, host_sets, kw, tokens_local = build_case(w, rank, world, device, args.exchange)
    peer_on = "shard" in kw and kw["shard"].peer is not None
    if peer_on and "--graph" not in sys.argv:
        args.graph = "on"
    if args.defer_weight_grad_reduce and "shard" in kw:
        kw["shard"].reduce_weight_grads = False
    if args.no_overlap_grad_reduce and "shard" in kw:
        kw["shard"].overlap_grad_reduce = False
    params = list(mod.parameters())
    video = "layers" in w
    if video:
        L = w["frame"]
        single = bool(w.get("single_pass"))
        split = lambda x: [x] if single else [x[:, f * L:(f + 1) * L].contiguous() for f in range(w["N"] // L)]
        dev_sets = [(split(x.to(device)), None) for x, _ in host_sets]
        if args.graph == "off" and "--graph" not in sys.argv:
            args.graph = "on"  # the frame loop is launch-bound from Python; the graph is the product path here

        def step(frames, _):
            if single:
                y = mod.forward_single_pass(frames[0], L)
                return y, [y]
            states, outs = None, []
            for f in frames:
                y, states = mod.frame_forward(f, states)
                outs.append(y)
            return outs[-1], outs
    else:
        dev_sets = [(x.to(device), gy.to(device)) for x, gy in host_sets]

        def step(x, gy):
            xr = x.requires_grad_(True)
            y = mod(xr, **kw)
            grads = torch.autograd.grad(y, [xr] + params, gy)
            return y, grads

    def sync_all():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- device-resident timing
    for i in range(args.warmup):
        step(*dev_sets[i % len(dev_sets)])
    sync_all()
    l0 = ops.launch_count()
    step(*dev_sets[0])
    launches_per_step = ops.launch_count() - l0
    use_graph = args.graph == "on"
    graphs = []
    if use_graph:
        # one graph per input set; kernels, memsets and NCCL collectives of a whole fwd+bwd step are captured
        sync_all()
        for xs_d, gy_d in dev_sets:
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                keep = step(xs_d, gy_d)
            graphs.append((g, keep))
        for g, _ in graphs:
            g.replay()
        sync_all()

    def run_step(i):
        if use_graph:
            graphs[i % len(graphs)][0].replay()
        else:
            step(*dev_sets[i % len(dev_sets)])

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sync_all()
    e0.record()
    for i in range(args.steps):
        run_step(i)
    e1.record()
    sync_all()
    launches = launches_per_step * args.steps
    clocks = sampler.stop() if rank == 0 else None
    ms_total = torch.tensor([e0.elapsed_time(e1)], device=device)
    if world > 1:
        dist.all_reduce(ms_total, op=dist.ReduceOp.MAX)
    ms_step = ms_total.item() / args.steps
    tokens_all = tokens_local * world
    value = tokens_all / (ms_step * 1e-3)
    # key-padding workload: `value` counts padded tokens; the fraction of valid context tokens is reported beside it
    valid_frac = float(kw["mask"].float().mean().item()) if torch.is_tensor(kw.get("mask")) else None

    # ---- end to end through the module API with host buffers (pinned), copies inside the timed region
    xs, gs = host_sets[0]
    y_host = torch.empty_like(xs).pin_memory()
    dx_host = torch.empty_like(xs).pin_memory()

    # Double-buffered: the host->device copy of step i+1 and the device->host copy of step i-1 run on their own
    # streams while the kernels of step i run; every step's copies are inside the timed region.
    copy_in, copy_out = torch.cuda.Stream(), torch.cuda.Stream()
    main = torch.cuda.current_stream()
    n_buf = 2
    xb = [torch.empty(xs.shape, dtype=xs.dtype, device=device) for _ in range(n_buf)]
    gb = None if video else [torch.empty(xs.shape, dtype=xs.dtype, device=device) for _ in range(n_buf)]
    ev_in = [torch.cuda.Event() for _ in range(n_buf)]
    ev_done = [None] * n_buf

    def stage_in(i):
        j = i % n_buf
        hx, hg = host_sets[i % len(host_sets)]
        with torch.cuda.stream(copy_in):
            if ev_done[j] is not None:
                copy_in.wait_event(ev_done[j])  # the step that last read this buffer
            xb[j].copy_(hx, non_blocking=True)
            if not video:
                gb[j].copy_(hg, non_blocking=True)
            ev_in[j].record(copy_in)

    def run_e2e(n):
        stage_in(0)
        for i in range(n):
            j = i % n_buf
            if i + 1 < n:
                stage_in(i + 1)
            main.wait_event(ev_in[j])
            if video:
                _, outs = step(split(xb[j]), None)
                results = ((torch.cat(outs, dim=1), y_host),)
            else:
                y, grads = step(xb[j].detach(), gb[j])
                results = ((y, y_host), (grads[0], dx_host))
            done = torch.cuda.Event()
            done.record(main)
            ev_done[j] = done
            with torch.cuda.stream(copy_out):
                copy_out.wait_event(done)
                for t, h in results:
                    h.copy_(t, non_blocking=True)
                    t.record_stream(copy_out)
        main.wait_stream(copy_out)

    e2e_steps = max(3, min(args.steps, 20))
    run_e2e(2)
    sync_all()
    e0.record()
    run_e2e(e2e_steps)
    e1.record()
    sync_all()
    ms_e2e = torch.tensor([e0.elapsed_time(e1)], device=device)
    if world > 1:
        dist.all_reduce(ms_e2e, op=dist.ReduceOp.MAX)
    e2e_val = tokens_all / (ms_e2e.item() / e2e_steps * 1e-3)
    h2d = (1 if video else 2) * xs.numel() * xs.element_size()
    d2h = (1 if video else 2) * xs.numel() * xs.element_size()

    # ---- roofline of the tensor-core kernel: per-launch CUDA-event timing of one instrumented step
    peaks = measured_peaks()
    # every rank runs the instrumented step (a token-sharded layer contains collectives); rank 0 reports
    roof = gemm_roofline(step, dev_sets, peaks, reps=2 if video else 5)
    sync_all()

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        v, sec, sample = cpu_reference_tokens_per_s(w, 3, 1)
        cpu = {"value": v, "unit": UNIT, "cores": torch.get_num_threads(), "kind": "port", "sample": sample}

    if rank == 0:
        status = _abi.read_status(device)
        line = {
            "metric": "pom_stack_fwd_tokens_per_s" if video else METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms_step, "higher_is_better": True,
            "scaling": "strong" if w["shard"] == "token" else "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": args.workload, "B_per_rank": w["B"], "N": w["N"], "D": w["D"], "degree": w["degree"],
                       "expand": w["expand"], "mask": w["mask"], "rope": w["rope"], "sharding": w["shard"],
                       "parallelism": f"{w['shard']}-shard x{world}",
                       "l2": "3 rotating input sets (>= 450 MB) plus ~1 GB of intermediates per step, larger than the 126 MB L2",
                       "e2e_pipeline": "double-buffered: H2D of step i+1 and D2H of step i-1 on their own streams beside the kernels of step i",
                       "valid_token_fraction": valid_frac,
                       "valid_tokens_per_s": None if valid_frac is None else value * valid_frac,
                       "cuda_graph": use_graph,
                       "exchange": ("peer-memory kernels" if peer_on else "nccl") if w["shard"] == "token" and world > 1 else None,
                       "weight_grad_allreduce_in_timed_region": bool(w["shard"] == "token" and world > 1
                                                                     and not args.defer_weight_grad_reduce)},
            "roofline": roof,
            "step_roofline": {"flops_per_step": flops_per_step(w) / (world if w["shard"] == "token" else 1),
                              "tflops": flops_per_step(w) / (world if w["shard"] == "token" else 1) / (ms_step * 1e-3) / 1e12,
                              "frac_of_burst_peak": flops_per_step(w) / (world if w["shard"] == "token" else 1) / (ms_step * 1e-3) / 1e12 / peaks["burst"],
                              "peak_source": peaks["source"]},
            "cpu_baseline": cpu,
            "e2e": {"value": e2e_val, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "ms_per_step": ms_e2e.item() / e2e_steps},
            "gpu_launches": launches,
            "clocks": clocks,
            "device_status": status,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def gemm_roofline(step, dev_sets, peaks, reps=5):
    """Times every tcgen05 GEMM launch of one step with CUDA events (on the launching stream) by wrapping the
    binding's GEMM entry points, and reports the launch that dominates the step."""
    from pom_b200 import functional, ops

    records = []
    originals = {}
    whole = functional.WHOLE_LAYER_CALLS
    functional.WHOLE_LAYER_CALLS = False  # same kernels, launched phase by phase so each can be bracketed by events

    def wrap(name, flops_of):
        fn = getattr(ops, name)
        originals[name] = fn

        def timed(*a, **k):
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            out = fn(*a, **k)
            e.record()
            records.append((name, flops_of(*a, **k), s, e))
            return out

        setattr(ops, name, timed)

    def gemm_flops(a, b, a_mn=False, b_mn=False, **_):
        M, K = (a.shape[1], a.shape[0]) if a_mn else (a.shape[0], a.shape[1])
        N = b.shape[1] if b_mn else b.shape[0]
        return 2.0 * M * N * K, f"gemm[{M}x{N}x{K}{' A^T' if a_mn else ''}{' B^T' if b_mn else ''}]"

    wrap("gemm", gemm_flops)
    wrap("ctx_gemm", lambda x, wpo, c, **_: (2.0 * x.shape[0] * x.shape[1] * x.shape[2] * wpo.shape[0], "ctx_gemm"))
    wrap("gate_gemm", lambda x, wse, b, h, **_: (2.0 * x.shape[0] * x.shape[1] * x.shape[2] * wse.shape[0], "gate_gemm"))
    wrap("gate_bwd_gemm", lambda dy, wo, *a, **_: (2.0 * dy.shape[0] * dy.shape[1] * dy.shape[2] * wo.shape[1], "gate_bwd_gemm"))
    try:
        for i in range(reps):
            step(*dev_sets[i % len(dev_sets)])
        torch.cuda.synchronize()
    finally:
        functional.WHOLE_LAYER_CALLS = whole
        for n, fn in originals.items():
            setattr(ops, n, fn)
    agg = {}
    for name, (fl, label), s, e in records:
        a = agg.setdefault(label, [0.0, 0.0, 0])
        a[0] += fl
        a[1] += s.elapsed_time(e)
        a[2] += 1
    rows = [{"kernel": k, "launches_per_step": v[2] / reps, "flops_per_launch": v[0] / v[2], "ms_per_launch": v[1] / v[2],
             "tflops": v[0] / v[1] / 1e9} for k, v in agg.items() if v[0] > 0]
    rows.sort(key=lambda r: -r["ms_per_launch"] * r["launches_per_step"])
    tot_fl = sum(v[0] for v in agg.values()) / reps
    tot_ms = sum(v[1] for v in agg.values()) / reps
    top = rows[0]
    return {"bound": "tensor", "kernel": "gemm_tcgen05_kernel: " + top["kernel"], "achieved": top["tflops"],
            "peak": peaks["burst"], "unit": "TFLOP/s", "frac": top["tflops"] / peaks["burst"],
            "peak_sustained": peaks["sustained"], "frac_of_sustained": top["tflops"] / peaks["sustained"],
            "peak_source": peaks["source"], "traffic": NCU_TRAFFIC_BYTES.get(top["kernel"]),
            "traffic_by_kernel": {k: v for k, v in NCU_TRAFFIC_BYTES.items()},
            "all_gemm_launches": {"tflops": tot_fl / tot_ms / 1e9, "ms_per_step": tot_ms, "frac": tot_fl / tot_ms / 1e9 / peaks["burst"]},
            "per_launch": rows}


if __name__ == "__main__":
    main()
