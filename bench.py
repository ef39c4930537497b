#!/usr/bin/env python
"""Benchmark of the PoM layer hot path (forward + backward) on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload dit|dit4k|masked|seq64k|seq64k_causal|...]
    python bench.py --impl reference ...        # CPU restatement of the reference path, same metric and config

One "step" is one forward + backward pass of one PoM layer over one batch of seeded synthetic
input, with gradients for the input and all four parameters.  Rank 0 prints one JSON line.

Workloads
  dit            B=32, N=1024 (32x32 patches), D=1152, degree 2, expand 2, bf16, no mask.  With
                 --gpus N every rank runs its own batch of 32 samples (weak scaling, no collective
                 on the data path: samples are independent).
  dit4k          the same token count as 8 samples of 4096 tokens (the headline sequence length).
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

The default run (workload dit) adds two records to its line: `headline_n4096` (the dit4k shape timed the same
way) and `token_shard` (seq64k and seq64k_causal: the 65536-token sequence sharded by token over the N ranks,
beside the same problem on one GPU timed in the same process; skip with --no-token-shard).
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
    "dit4k": dict(B=8, N=4096, D=1152, degree=2, expand=2, mask="none", rope=None, shard="batch"),
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
N_INPUT_SETS = 3

# DRAM bytes (read + write) of one launch from an ncu capture of the kernel as shipped (dram__bytes_read.sum +
# dram__bytes_write.sum); launches without a capture report null beside their algorithmic bytes.
NCU_TRAFFIC_BYTES = {
    "gemm[32768x1152x4608 B^T]": 399.2e6,
}


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        d = json.load(open(path))
        return dict(hbm=d["hbm_gbs"], burst=d["bf16_tflops"], sustained=d.get("bf16_tflops_sustained", d["bf16_tflops"]),
                    source="measured")
    return dict(hbm=6650.0, burst=1590.0, sustained=1400.0, source="fallback")


def workload_config(name, w, world):
    """The `config` object of the JSON line: the same for the B200 arm and the CPU reference arm."""
    return {"workload": name, "B_per_rank": w["B"], "N": w["N"], "D": w["D"], "degree": w["degree"],
            "expand": w["expand"], "mask": w["mask"], "rope": w["rope"], "sharding": w["shard"],
            "parallelism": f"{w['shard']}-shard x{world}",
            "l2": f"{N_INPUT_SETS} rotating input sets; inputs plus per-step intermediates (~1 GB) exceed the 126 MB L2"}


class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi while the timed regions run."""
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        # nvidia-smi numbers GPUs by PCI bus id, CUDA by its own order: name the GPU by its bus id where possible
        try:
            p = torch.cuda.get_device_properties(index)
            index = f"{p.pci_domain_id:08x}:{p.pci_bus_id:02x}:{p.pci_device_id:02x}.0"
        except Exception:
            pass
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
        sm, mx, pw, reasons = [], [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            if len(r) < 7:
                continue
            try:
                sm.append(float(r[0]))
                mx.append(float(r[1]))
                pw.append(float(r[2]))
            except ValueError:
                continue
            for n, v in zip(names, r[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        # "under load": samples drawing clearly more than the idle power of the board
        busy = [s for s, p in zip(sm, pw) if p > 350.0]
        return {"sm_mhz": statistics.median(busy or sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm), "samples_under_load": len(busy),
                "power_w_max": max(pw) if pw else None}


def bind_to_gpu_numa_node(local_rank):
    """Pins this process to the CPUs of the NUMA node its GPU hangs off, before any pinned host buffer is
    allocated: first touch then places the staging pages on that node and the copy threads run beside them.
    Returns a short description (None when the topology cannot be read; nothing is changed then)."""
    try:
        p = torch.cuda.get_device_properties(local_rank)
        bus = f"{p.pci_domain_id:04x}:{p.pci_bus_id:02x}:{p.pci_device_id:02x}.0"
    except Exception:
        return None
    cpus, how = set(), None
    try:
        node = int(open(f"/sys/bus/pci/devices/{bus}/numa_node").read().strip())
        if node >= 0:
            for part in open(f"/sys/devices/system/node/node{node}/cpulist").read().strip().split(","):
                lo, _, hi = part.partition("-")
                cpus.update(range(int(lo), int(hi or lo) + 1))
            how = f"numa node {node} (sysfs)"
    except Exception:
        cpus = set()
    if not cpus:
        # containers often hide the PCI device's numa_node: the driver's own CPU affinity mask of the GPU (a read)
        try:
            import pynvml

            pynvml.nvmlInit()
            h = pynvml.nvmlDeviceGetHandleByPciBusId(bus.encode())
            words = pynvml.nvmlDeviceGetCpuAffinity(h, (os.cpu_count() + 63) // 64)
            for i, w in enumerate(words):
                cpus.update(64 * i + b for b in range(64) if (int(w) >> b) & 1)
            how = "cpu affinity of the GPU (NVML)"
        except Exception:
            cpus = set()
    try:
        allowed = cpus & os.sched_getaffinity(0)
        if not allowed or allowed == os.sched_getaffinity(0):
            return None
        os.sched_setaffinity(0, allowed)
        return f"{how}, {len(allowed)} cpus"
    except Exception:
        return None


def flops_per_step(w):
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
def cpu_reference_tokens_per_s(w, steps, warmup, max_tokens=65536):
    """Times the CPU restatement of the reference path (oracle/pom_oracle.py, fp32, all host threads) on the
    workload's own shape when it has at most `max_tokens` tokens per step, else on a sample of it with the batch cut
    down to that many tokens.  Inputs rotate over N_INPUT_SETS sets like the B200 arm's."""
    from oracle import pom_oracle as O

    torch.set_num_threads(os.cpu_count() or 1)
    D, K, E = w["D"], w["degree"], w["expand"]
    if "layers" in w:
        return cpu_reference_video(w, steps, warmup, O)
    B, N = w["B"], w["N"]
    full = B * N <= max_tokens
    if not full:
        B = max(1, max_tokens // N)
        N = min(N, max_tokens)
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
    sets = [(torch.randn(B, N, D, generator=g).requires_grad_(True), torch.randn(B, N, D, generator=g))
            for _ in range(N_INPUT_SETS)]
    if w["mask"] == "keypad":
        L = torch.randint(256, N + 1, (B,), generator=g)
        kw["mask"] = (torch.arange(N).view(1, N) < L.view(B, 1)).float()
    elif w["mask"] == "causal":
        kw["mask"] = "causal"

    def step(i):
        x, gy = sets[i % N_INPUT_SETS]
        y = model.forward(x, **kw)
        torch.autograd.grad(y, [x] + model.parameters(), gy)

    for i in range(warmup):
        step(i)
    times = []
    for i in range(steps):
        t0 = time.perf_counter()
        step(i)
        times.append(time.perf_counter() - t0)
    sec = statistics.median(times)
    what = "the full workload shape" if full else "a sample of the workload"
    return (B * N) / sec, sec, f"{what}: B={B}, N={N} (fp32, {torch.get_num_threads()} threads), median of {steps} steps"


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


def run_reference(args, w, rank, world):
    """CPU arm: rank 0 alone runs the oracle port with all host threads, on the B200 arm's config."""
    if rank != 0:
        return
    steps, warmup = max(1, args.steps), max(0, args.warmup)
    # keep the whole run within a few minutes whatever --steps says: probe one step, then cap
    t0 = time.perf_counter()
    cpu_reference_tokens_per_s(w, 1, 0)
    probe = time.perf_counter() - t0
    budget = 150.0
    if (steps + warmup) * probe > budget:
        warmup = min(warmup, 1)
        steps = max(1, min(steps, int(budget / probe) - warmup))
    val, sec, sample = cpu_reference_tokens_per_s(w, steps, warmup)
    line = {
        "impl": "reference", "metric": METRIC, "value": val, "unit": UNIT, "n_gpus": args.gpus, "steps": steps,
        "warmup": warmup, "ms_per_step": sec * 1e3, "higher_is_better": True,
        "scaling": "strong" if w["shard"] == "token" else "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(args.workload, w, world),
        "cpu_baseline": {"value": val, "unit": UNIT, "cores": torch.get_num_threads(), "kind": "port", "sample": sample},
        "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------- B200 arm
def build_case(w, rank, world, device, exchange="nccl", peer=None):
    """Module, rotating pinned input sets and call kwargs for this rank."""
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
                     for _ in range(N_INPUT_SETS)]
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
            kw["shard"] = SeqShard(token_offset=off, n_global=N, peer=peer if exchange == "peer" else None)
        tokens_local = B * n_loc
    else:
        n_loc = N
        tokens_local = B * N
    if w["mask"] == "causal":
        kw["mask"] = "causal"
    gen = torch.Generator().manual_seed(1000 + rank)
    host_sets = []
    for _ in range(N_INPUT_SETS):
        x = torch.randn(B, n_loc, D, generator=gen).to(torch.bfloat16).pin_memory()
        gy = torch.randn(B, n_loc, D, generator=gen).to(torch.bfloat16).pin_memory()
        host_sets.append((x, gy))
    if w["mask"] == "keypad":
        L = torch.randint(256, N + 1, (B,), generator=gen)
        kw["mask"] = (torch.arange(N).view(1, N) < L.view(B, 1)).float().to(device)
    return mod, host_sets, kw, tokens_local


def make_peer(w, world, device, rank):
    """Peer-memory exchange buffers for the token-sharded workloads (collective); None when the ranks cannot map
    each other's memory, in which case every rank falls back to NCCL together."""
    import torch.distributed as dist
    from pom_b200.peer import PeerExchange

    P = w["D"] * w["expand"]
    n_params = 2 * P * w["D"] + w["D"] * P + P + P * w["degree"]
    peer = None
    try:
        peer = PeerExchange(slot_floats=max(4096, w["B"] * P), flat_floats=n_params + 4)
        ok = torch.ones(1, device=device)
    except Exception as e:  # e.g. CUDA IPC not permitted between these processes
        print(f"[bench] peer exchange unavailable on rank {rank}: {e}; using NCCL", file=sys.stderr)
        ok = torch.zeros(1, device=device)
    dist.all_reduce(ok, op=dist.ReduceOp.MIN)
    return peer if float(ok.item()) != 0.0 else None


class Case:
    """One workload on this rank: module, device-resident input sets and a step function, optionally replayed
    from CUDA graphs (one per input set)."""

    def __init__(self, name, w, rank, world, device, exchange="nccl", peer=None, graph=False):
        from pom_b200 import ops

        self.name, self.w, self.world, self.device = name, w, world, device
        self.mod, self.host_sets, self.kw, self.tokens_local = build_case(w, rank, world, device, exchange, peer)
        self.params = list(self.mod.parameters())
        self.video = "layers" in w
        self.peer_on = "shard" in self.kw and self.kw["shard"].peer is not None
        if self.video:
            L = w["frame"]
            self.single = bool(w.get("single_pass"))
            self.split = lambda x: [x] if self.single else [x[:, f * L:(f + 1) * L].contiguous()
                                                           for f in range(w["N"] // L)]
            self.dev_sets = [(self.split(x.to(device)), None) for x, _ in self.host_sets]
        else:
            self.dev_sets = [(x.to(device), gy.to(device)) for x, gy in self.host_sets]
        self.graphs = []
        self.use_graph = graph
        self.ops = ops
        self.launches_per_step = 0

    def step(self, x, gy):
        if self.video:
            if self.single:
                y = self.mod.forward_single_pass(x[0], self.w["frame"])
                return y, [y]
            states, outs = None, []
            for f in x:
                y, states = self.mod.frame_forward(f, states)
                outs.append(y)
            return outs[-1], outs
        xr = x.requires_grad_(True)
        y = self.mod(xr, **self.kw)
        grads = torch.autograd.grad(y, [xr] + self.params, gy)
        return y, grads

    def prepare(self, warmup, sync_all):
        for i in range(warmup):
            self.step(*self.dev_sets[i % len(self.dev_sets)])
        sync_all()
        l0 = self.ops.launch_count()
        self.step(*self.dev_sets[0])
        self.launches_per_step = self.ops.launch_count() - l0
        if self.use_graph:
            sync_all()
            for xs_d, gy_d in self.dev_sets:
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g):
                    keep = self.step(xs_d, gy_d)
                self.graphs.append((g, keep))
            for g, _ in self.graphs:
                g.replay()
        sync_all()

    def run(self, i):
        if self.use_graph:
            self.graphs[i % len(self.graphs)][0].replay()
        else:
            self.step(*self.dev_sets[i % len(self.dev_sets)])

    def timed(self, steps, reps, sync_all, reduce_max):
        """`reps` repetitions of exactly `steps` steps, each bracketed by barrier + synchronize and timed with CUDA
        events on the launching stream; every repetition is the max over ranks.  Returns ms per step per repetition."""
        out = []
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        for _ in range(reps):
            sync_all()
            e0.record()
            for i in range(steps):
                self.run(i)
            e1.record()
            sync_all()
            out.append(reduce_max(e0.elapsed_time(e1)) / steps)
        return out

    def timed_with_grad_allreduce(self, steps, reps, sync_all, reduce_max, overlap=True):
        """Data-parallel form of the batch-sharded step: as `timed`, plus an NCCL sum of every parameter gradient over
        the ranks inside the timed region, on a side stream so that it runs beside the next step's kernels (what
        DistributedDataParallel does with its buckets).  Returns (ms per step per repetition, bytes reduced per step)."""
        import torch.distributed as dist

        main, side = torch.cuda.current_stream(), torch.cuda.Stream()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        out, nbytes = [], 0
        for rep in range(-1, reps):  # repetition -1: three untimed steps (first use of the collective on this stream)
            sync_all()
            e0.record()
            for i in range(steps if rep >= 0 else 3):
                _, grads = self.step(*self.dev_sets[i % len(self.dev_sets)])
                # the layer returns its parameter gradients as views of one flat buffer: one collective for all
                base = grads[1]._base
                bufs = [base] if base is not None and all(g._base is base for g in grads[1:]) else list(grads[1:])
                if overlap:
                    side.wait_stream(main)
                with torch.cuda.stream(side if overlap else main):
                    for g in bufs:
                        dist.all_reduce(g)
                        if overlap:
                            g.record_stream(side)
                nbytes = sum(g.numel() * g.element_size() for g in bufs)
            main.wait_stream(side)
            e1.record()
            sync_all()
            if rep >= 0:
                out.append(reduce_max(e0.elapsed_time(e1)) / steps)
        return out, nbytes

    def timed_with_peer_grad_sum(self, peer, steps, reps, sync_all, reduce_max):
        """The data-parallel step with the library's own exchange: the backward pass of the layer accumulates the
        parameter gradients in the peer-mapped region and sums them over the ranks itself (bf16 on the wire, the
        all-reduce kernel also does the rounding that a cast kernel does otherwise).  Nothing else is added."""
        self.kw["grad_peer"] = peer
        try:
            for i in range(3):
                self.step(*self.dev_sets[i % len(self.dev_sets)])
            return self.timed(steps, reps, sync_all, reduce_max)
        finally:
            del self.kw["grad_peer"]

    def release(self):
        self.graphs = []
        self.dev_sets = []
        self.host_sets = []
        self.mod = None


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--reps", type=int, default=10,
                    help="repetitions of the timed region of --steps steps; ms_per_step is their median")
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default="dit", choices=sorted(WORKLOADS))
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-token-shard", action="store_true",
                    help="default workload: skip the token-sharded 64 k-token records")
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
        run_reference(args, w, rank, world)
        return

    if os.environ.get("NCCL_DEBUG", "").upper() == "VERSION":
        os.environ["NCCL_DEBUG"] = "WARN"  # keep stdout to the one JSON line
    import torch.distributed as dist
    from pom_b200 import _abi

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the B200 arm has no CPU path (use --impl reference for the CPU arm)")
    all_cpus = os.sched_getaffinity(0)
    numa = bind_to_gpu_numa_node(local_rank)
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
    args.reps = max(args.reps, 1)

    def sync_all():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def reduce_max(ms):
        if world == 1:
            return ms
        t = torch.tensor([ms], device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return t.item()

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()  # runs from before the warm-up until after the end-to-end leg

    peaks = measured_peaks()
    token = w["shard"] == "token"
    peer = make_peer(w, world, device, rank) if (token and world > 1 and args.exchange == "peer") else None
    graph_flag_given = "--graph" in sys.argv
    graph = args.graph == "on" or ((peer is not None or "layers" in w) and not graph_flag_given)
    case = Case(args.workload, w, rank, world, device, args.exchange, peer, graph)
    if args.defer_weight_grad_reduce and "shard" in case.kw:
        case.kw["shard"].reduce_weight_grads = False
    if args.no_overlap_grad_reduce and "shard" in case.kw:
        case.kw["shard"].overlap_grad_reduce = False
    video = case.video

    # ---- device-resident timing
    case.prepare(args.warmup, sync_all)
    per_rep = case.timed(args.steps, args.reps, sync_all, reduce_max)
    ms_step = statistics.median(per_rep)
    launches = case.launches_per_step * args.steps
    tokens_all = case.tokens_local * world
    value = tokens_all / (ms_step * 1e-3)
    # key-padding workload: `value` counts padded tokens; the fraction of valid context tokens is reported beside it
    valid_frac = float(case.kw["mask"].float().mean().item()) if torch.is_tensor(case.kw.get("mask")) else None

    # ---- the same batch-sharded step as data-parallel training: parameter gradients summed over the ranks
    data_parallel = None
    if world > 1 and not token and not video:
        dp_rep, dp_bytes = case.timed_with_grad_allreduce(args.steps, min(args.reps, 5), sync_all, reduce_max)
        dp_ms = statistics.median(dp_rep)
        data_parallel = {
            "ms_per_step": dp_ms, "ms_per_step_min": min(dp_rep), "ms_per_step_max": max(dp_rep),
            "tokens_per_s": tokens_all / (dp_ms * 1e-3), "reps": len(dp_rep),
            "grad_allreduce": "one NCCL sum of the flat bf16 parameter-gradient buffer over the ranks inside the timed "
                              "region, on a side stream beside the next step's kernels",
            "grad_bytes_per_rank_and_step": dp_bytes,
        }
        dp_peer = make_peer(w, world, device, rank) if args.exchange == "peer" else None
        pr = None
        if dp_peer is not None:
            try:
                pr = case.timed_with_peer_grad_sum(dp_peer, args.steps, min(args.reps, 5), sync_all, reduce_max)
            except NotImplementedError as e:  # raised on every rank alike, before anything is launched
                data_parallel["peer_kernels"] = {"unavailable": str(e)}
        if pr is not None:
            pm = statistics.median(pr)
            data_parallel["peer_kernels"] = {
                "ms_per_step": pm, "ms_per_step_min": min(pr), "ms_per_step_max": max(pr),
                "tokens_per_s": tokens_all / (pm * 1e-3), "reps": len(pr),
                "grad_allreduce": "inside the layer's backward pass: fp32 accumulators in the peer-mapped region, summed "
                                  "over the ranks by the library's all-reduce kernel with bf16 on the wire",
                "peer_status_max_over_ranks": int(reduce_max(float(abs(_abi.read_status(device))))),
            }
        if dp_peer is not None:
            sync_all()
            dp_peer.close()

    # ---- end to end through the module API with host buffers (pinned), copies inside the timed region
    e2e = measure_e2e(case, args, device, world, sync_all, reduce_max)

    # ---- roofline of the tensor-core kernel: per-launch CUDA-event timing of one instrumented step
    # every rank runs the instrumented step (a token-sharded layer contains collectives); rank 0 reports
    roof = gemm_roofline(case.step, case.dev_sets, peaks, reps=2 if video else 5)
    sync_all()
    clocks = sampler.stop() if rank == 0 else None

    headline = None
    shard_rec = None
    if args.workload == "dit":
        case.release()
        torch.cuda.empty_cache()
        headline = measure_headline(args, rank, world, device, sync_all, reduce_max, peaks)
        if not args.no_token_shard:
            shard_rec = measure_token_shard(args, rank, world, device, sync_all, reduce_max, peaks)

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        os.sched_setaffinity(0, all_cpus)  # the CPU leg may use every core the process was given
        v, sec, sample = cpu_reference_tokens_per_s(w, 3, 1)
        cpu = {"value": v, "unit": UNIT, "cores": torch.get_num_threads(), "kind": "port", "sample": sample}

    if rank == 0:
        status = _abi.read_status(device)
        fl = flops_per_step(w) / (world if token else 1)
        config = workload_config(args.workload, w, world)
        config.update({
            "e2e_pipeline": "double-buffered: H2D of step i+1 and D2H of step i-1 on their own streams beside the kernels of step i",
            "valid_token_fraction": valid_frac,
            "valid_tokens_per_s": None if valid_frac is None else value * valid_frac,
            "cuda_graph": case.use_graph,
            "exchange": ("peer-memory kernels" if case.peer_on else "nccl") if token and world > 1 else None,
            "weight_grad_allreduce_in_timed_region": bool(token and world > 1 and not args.defer_weight_grad_reduce),
            "host_affinity": numa,
        })
        line = {
            "metric": "pom_stack_fwd_tokens_per_s" if video else METRIC, "value": value, "unit": UNIT, "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step,
            "ms_per_step_min": min(per_rep), "ms_per_step_max": max(per_rep), "reps": args.reps,
            "higher_is_better": True, "scaling": "strong" if token else "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": config,
            "roofline": roof,
            "step_roofline": {"flops_per_step": fl, "tflops": fl / (ms_step * 1e-3) / 1e12,
                              "frac_of_burst_peak": fl / (ms_step * 1e-3) / 1e12 / peaks["burst"],
                              "peak_source": peaks["source"]},
            "headline_n4096": headline,
            "data_parallel": data_parallel,
            "token_shard": shard_rec,
            "cpu_baseline": cpu,
            "e2e": e2e,
            "gpu_launches": launches,
            "clocks": clocks,
            "device_status": status,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def measure_e2e(case, args, device, world, sync_all, reduce_max):
    """The same metric through the module API with pinned host buffers: every step's inputs cross PCIe host to
    device and its outputs (y, dx) device to host inside the timed region.  Double-buffered: the host->device copy
    of step i+1 and the device->host copy of step i-1 run on their own streams while the kernels of step i run."""
    video = case.video
    xs, _ = case.host_sets[0]
    y_host = torch.empty_like(xs).pin_memory()
    dx_host = torch.empty_like(xs).pin_memory()
    copy_in, copy_out = torch.cuda.Stream(), torch.cuda.Stream()
    main_stream = torch.cuda.current_stream()
    n_buf = 2
    xb = [torch.empty(xs.shape, dtype=xs.dtype, device=device) for _ in range(n_buf)]
    gb = None if video else [torch.empty(xs.shape, dtype=xs.dtype, device=device) for _ in range(n_buf)]
    ev_in = [torch.cuda.Event() for _ in range(n_buf)]
    ev_done = [None] * n_buf

    def stage_in(i):
        j = i % n_buf
        hx, hg = case.host_sets[i % len(case.host_sets)]
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
            main_stream.wait_event(ev_in[j])
            if video:
                _, outs = case.step(case.split(xb[j]), None)
                results = ((torch.cat(outs, dim=1), y_host),)
            else:
                y, grads = case.step(xb[j].detach(), gb[j])
                results = ((y, y_host), (grads[0], dx_host))
            done = torch.cuda.Event()
            done.record(main_stream)
            ev_done[j] = done
            with torch.cuda.stream(copy_out):
                copy_out.wait_event(done)
                for t, h in results:
                    h.copy_(t, non_blocking=True)
                    t.record_stream(copy_out)
        main_stream.wait_stream(copy_out)

    e2e_steps = max(3, min(args.steps, 20))
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    run_e2e(2)
    sync_all()
    e0.record()
    run_e2e(e2e_steps)
    e1.record()
    sync_all()
    ms = reduce_max(e0.elapsed_time(e1)) / e2e_steps
    h2d = (1 if video else 2) * xs.numel() * xs.element_size()
    d2h = (1 if video else 2) * xs.numel() * xs.element_size()
    return {"value": case.tokens_local * world / (ms * 1e-3), "unit": UNIT, "h2d_bytes_per_step": h2d,
            "d2h_bytes_per_step": d2h, "ms_per_step": ms, "steps": e2e_steps,
            "copy_gbs_per_rank_each_way": h2d / (ms * 1e-3) / 1e9}


def measure_headline(args, rank, world, device, sync_all, reduce_max, peaks):
    """The layer at the headline sequence length: D=1152, degree 2, expand 2, N=4096, B=8 per rank (the same
    32768 tokens per step as the dit workload), timed exactly like `value`."""
    w = dict(WORKLOADS["dit4k"])
    case = Case("dit4k", w, rank, world, device)
    case.prepare(args.warmup, sync_all)
    per_rep = case.timed(args.steps, max(3, args.reps // 2), sync_all, reduce_max)
    ms = statistics.median(per_rep)
    fl = flops_per_step(w)
    rec = {"config": workload_config("dit4k", w, world), "ms_per_step": ms, "ms_per_step_min": min(per_rep),
           "ms_per_step_max": max(per_rep), "tokens_per_s": case.tokens_local * world / (ms * 1e-3),
           "tflops_per_gpu": fl / (ms * 1e-3) / 1e12, "frac_of_burst_peak": fl / (ms * 1e-3) / 1e12 / peaks["burst"],
           "peak_source": peaks["source"]}
    case.release()
    torch.cuda.empty_cache()
    return rec


def measure_token_shard(args, rank, world, device, sync_all, reduce_max, peaks):
    """Strong scaling of one 65536-token sequence (2-D rotary, non-causal and token-causal) sharded by token over
    the `world` ranks: ms/step of the sharded step (parameter-gradient all-reduce inside the timed region), the
    same problem on one GPU timed on rank 0 in this process, and their ratio."""
    import torch.distributed as dist
    from pom_b200 import _abi

    out = {}
    steps = max(5, min(args.steps, 50))
    reps = max(3, args.reps // 2)
    solo_sync = torch.cuda.synchronize
    peer = None
    if world > 1 and args.exchange == "peer":
        peer = make_peer(WORKLOADS["seq64k"], world, device, rank)
    for name in ("seq64k", "seq64k_causal"):
        w = dict(WORKLOADS[name])
        fl = flops_per_step(w)
        rec = {"config": workload_config(name, w, world), "n_gpus": world, "steps": steps, "reps": reps,
               "flops_per_step": fl}
        # one GPU, whole sequence, on rank 0 (the other ranks wait at the barrier below)
        ms1 = 0.0
        if rank == 0:
            solo = Case(name, w, 0, 1, device)
            solo.prepare(args.warmup, solo_sync)
            r1 = solo.timed(steps, reps, solo_sync, lambda ms: ms)
            ms1 = statistics.median(r1)
            rec["launches_per_step_1gpu"] = solo.launches_per_step
            solo.release()
            torch.cuda.empty_cache()
        if world > 1:
            t = torch.tensor([ms1], device=device)
            dist.broadcast(t, 0)
            ms1 = t.item()
        rec["ms_per_step_1gpu"] = ms1
        rec["frac_of_burst_peak_1gpu"] = fl / (ms1 * 1e-3) / 1e12 / peaks["burst"]
        if world > 1:
            sh = Case(name, w, rank, world, device, args.exchange, peer, graph=peer is not None)
            sh.prepare(args.warmup, sync_all)
            rs = sh.timed(steps, reps, sync_all, reduce_max)
            msn = statistics.median(rs)
            rec.update({"ms_per_step_sharded": msn, "ms_per_step_sharded_min": min(rs),
                        "ms_per_step_sharded_max": max(rs), "speedup_vs_1gpu": ms1 / msn,
                        "tokens_per_s": w["B"] * w["N"] / (msn * 1e-3),
                        "frac_of_burst_peak_per_gpu": fl / world / (msn * 1e-3) / 1e12 / peaks["burst"],
                        "transport": "peer-memory kernels inside one CUDA graph per rank" if sh.peer_on else "nccl, eager",
                        "weight_grad_allreduce_in_timed_region": True,
                        "launches_per_step_per_rank": sh.launches_per_step})
            sh.release()
            torch.cuda.empty_cache()
            st = torch.tensor([float(_abi.read_status(device))], device=device)
            dist.all_reduce(st, op=dist.ReduceOp.MAX)
            rec["peer_status_max_over_ranks"] = int(st.item())
        else:
            rec["tokens_per_s"] = w["B"] * w["N"] / (ms1 * 1e-3)
        out[name] = rec
    if peer is not None:
        peer.close()
    return out


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

    def gemm_flops(a, b, a_mn=False, b_mn=False, out=None, accumulate=False, **_):
        M, K = (a.shape[1], a.shape[0]) if a_mn else (a.shape[0], a.shape[1])
        N = b.shape[1] if b_mn else b.shape[0]
        nbytes = 2.0 * (M * K + N * K) + M * N * (4.0 if accumulate or (out is not None and out.dtype == torch.float32) else 2.0)
        return 2.0 * M * N * K, f"gemm[{M}x{N}x{K}{' A^T' if a_mn else ''}{' B^T' if b_mn else ''}]", nbytes

    def phase(label, n_out):
        # operands A (M x D) and B (P x D) read once; n_out bf16 (M x P) tensors written (and z re-read in backward)
        def f(x, wgt, *a, **k):
            M, D = x.shape[0] * x.shape[1], x.shape[2]
            P = wgt.shape[0] if label != "gate_bwd_gemm" else wgt.shape[1]
            tag = label + ("+rope" if k.get("rope") is not None else "")
            return 2.0 * M * D * P, tag, 2.0 * (M * D + P * D) + 2.0 * n_out * M * P
        return f

    wrap("gemm", gemm_flops)
    wrap("ctx_gemm", phase("ctx_gemm", 1))
    wrap("gate_gemm", phase("gate_gemm", 2))
    wrap("gate_bwd_gemm", phase("gate_bwd_gemm", 2))
    try:
        for i in range(reps):
            step(*dev_sets[i % len(dev_sets)])
        torch.cuda.synchronize()
    finally:
        functional.WHOLE_LAYER_CALLS = whole
        for n, fn in originals.items():
            setattr(ops, n, fn)
    agg = {}
    for name, (fl, label, nbytes), s, e in records:
        a = agg.setdefault(label, [0.0, 0.0, 0, nbytes])
        a[0] += fl
        a[1] += s.elapsed_time(e)
        a[2] += 1
    rows = [{"kernel": k, "launches_per_step": v[2] / reps, "flops_per_launch": v[0] / v[2], "ms_per_launch": v[1] / v[2],
             "tflops": v[0] / v[1] / 1e9, "algorithmic_bytes": v[3], "ncu_dram_bytes": NCU_TRAFFIC_BYTES.get(k)}
            for k, v in agg.items() if v[0] > 0]
    rows.sort(key=lambda r: -r["ms_per_launch"] * r["launches_per_step"])
    tot_fl = sum(v[0] for v in agg.values()) / reps
    tot_ms = sum(v[1] for v in agg.values()) / reps
    top = rows[0]
    return {"bound": "tensor", "kernel": "gemm_tcgen05_2cta_kernel: " + top["kernel"], "achieved": top["tflops"],
            "peak": peaks["burst"], "unit": "TFLOP/s", "frac": top["tflops"] / peaks["burst"],
            "peak_sustained": peaks["sustained"], "frac_of_sustained": top["tflops"] / peaks["sustained"],
            "peak_source": peaks["source"], "traffic": top["ncu_dram_bytes"],
            "algorithmic_bytes": top["algorithmic_bytes"],
            "all_gemm_launches": {"tflops": tot_fl / tot_ms / 1e9, "ms_per_step": tot_ms, "frac": tot_fl / tot_ms / 1e9 / peaks["burst"]},
            "per_launch": rows}


if __name__ == "__main__":
    main()
