"""Benchmark of the hot path: Gated DeltaNet chunk forward + backward at BASELINE config 1.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload gdn|ssd|kda]

One step = one forward + backward of ``ops.linear_attention("gated_deltanet", ...)`` over one batch
(B=8, T=2048, H=16, K=V=128, bf16 q/k/v/dO, fp32 gates, packed documents of uniform length 64-2048 as
``segment_ids``), for a fixed output cotangent, as the reference's kernel benchmark defines ``fwd+bwd``
(``benchmarks/harness.py:98-118``). Inputs are seeded synthetic tensors (the reference benches this path on
synthetic tensors too). With N > 1 (``torchrun``) every rank runs the same workload on its own GPU and its own
seed: the batch x heads axis shards with no communication, so the scaling is weak and ``value`` is the aggregate.

Printed JSON (one line, rank 0): tokens/s with inputs resident in HBM (``value``), the same through the public
API from pinned host buffers (``e2e``), the roofline position of the dominant kernel (per-kernel CUDA-event
times recorded by the library inside the timed region), SM clocks sampled during the timed region, and a CPU
baseline (the oracle port of the reference's chunked algorithm, timed on this host's cores on a bounded sample).
``--impl reference`` times that CPU port alone (the reference's own JAX CPU path cannot run here: JAX is not
installed on the image).
"""

from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import numpy as np  # noqa: E402
import torch  # noqa: E402

METRIC = "GDN chunk fwd+bwd tokens/s/GPU (B8·T2048·H16·d128 bf16); % bf16 TC peak"
CHUNK = 64

WORKLOADS = {
    "gdn": dict(name="config1: gated_deltanet B8 T2048 H16 K128 V128 chunk64 bf16, packed docs U[64,2048]", index=1),
    "ssd": dict(name="config2: mamba2 SSD B8 T2048 H64 P64 N128 G1 bf16", index=2),
    "kda": dict(name="config3: kda B4 T4096 H16 K128 V128 bf16, packed docs U[128,4096]", index=3),
    "longctx": dict(name="config4: gated_deltanet B1 T1064960 H16 K128 V128 bf16, packed docs U[4096,131072], "
                         "sequence-parallel over the ranks", index=4),
}
METRICS = {
    "gdn": None,  # the headline metric
    "ssd": "Mamba-2 SSD chunk fwd+bwd tokens/s (B8·T2048·H64·P64·N128 bf16)",
    "kda": "KDA fwd+bwd tokens/s (B4·T4096·H16·d128 bf16)",
    "longctx": "GDN fwd+bwd tokens/s on one 1,064,960-token sequence (H16·d128 bf16), sequence-parallel",
}
LONG_T = 1_064_960


def peaks() -> dict:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return dict(hbm_gbs=d["hbm_gbs"], bf16_tflops=d["bf16_tflops"], source="measured")
    return dict(hbm_gbs=6650.0, bf16_tflops=1590.0, source="fallback")


# Algorithmic work of each kernel per (chunk, head) at K = V = 128, bf16 (bytes it must read + write once; MACs
# of its products excluding recomputation and the triangular inverse). 1 MAC = 2 FLOP.
def kernel_model(K: int, V: int, delta: bool, save: bool) -> dict:
    e = 2
    qk, vv, st, cc = 64 * K * e, 64 * V * e, K * V * e, 64 * 64 * e
    gates = 128 * 4 + 64
    m = {}
    if delta:
        m["kkt_inv"] = dict(bytes=qk + gates + 2 * cc, mac=64 * 64 * K)  # writes T0 and its gated form Ag
    m["sg_fwd"] = dict(bytes=2 * qk + vv + (cc if delta else 0) + gates + vv + (st + (2 * vv if delta else 0) if save else 0),  # residuals h, Vn, W
                       mac=64 * 64 * K + 64 * 64 * V * (2 if delta else 1) + K * V * 64 * (3 if delta else 2))
    m["sg_bwd_state"] = dict(bytes=2 * qk + vv + (cc if delta else 0) + gates + st + vv + (vv if delta else 0),
                             mac=64 * K * V + 64 * 64 * V * (2 if delta else 1) + K * V * 64 * (2 if delta else 1))
    # tcgen05 path (K = V = 128): the chunk gradients are two kernels, dP and a dG partial go through the scratch
    m["sg_grads_q"] = dict(bytes=2 * vv + st + 2 * qk + gates + cc + qk + 256,
                           mac=64 * 64 * V + 64 * K * V + 64 * 64 * K)
    m["sg_grads_k"] = dict(
        bytes=2 * qk + cc + 2 * st + gates + 256 + qk + ((4 * vv + cc) if delta else vv),
        mac=64 * 64 * K + 64 * K * V + ((64 * 64 * V + 64 * 64 * K + 2 * 64 ** 3 + 2 * 64 * 64 * K + 64 * K * V) if delta else 0))
    m["sg_chunk_grads"] = dict(
        bytes=2 * qk + 2 * vv + 2 * st + gates + 2 * qk + ((cc + 3 * vv) if delta else 0),
        mac=64 * 64 * V + 64 * K * V + 64 * 64 * K * 2 + 64 * K * V + ((64 * 64 * V + 64 * K * V + 2 * 64 * 64 * K) if delta else 0))
    # KDA (per-channel gates): the gate-folded operands go through HBM between the prologue and the state passes, and
    # the gradients of the folded state-side operands between the two gradient kernels (fp32)
    f32 = 64 * K * 4
    m["kda_prep"] = dict(bytes=2 * qk + f32 + 3 * qk + 3 * cc + K * 4 + gates, mac=2 * 64 * 64 * K)
    m["kda_fwd"] = dict(bytes=3 * qk + 2 * cc + vv + K * 4 + vv + (st + 2 * vv if save else 0),
                        mac=64 * 64 * V * 2 + K * V * 64 * 3)
    m["kda_bwd_state"] = dict(bytes=3 * qk + 2 * cc + vv + K * 4 + st + 2 * vv, mac=64 * K * V + 64 * 64 * V * 2 + K * V * 64 * 2)
    m["kda_chunk_grads"] = dict(bytes=2 * vv + 2 * st + 3 * vv + 3 * f32 + 2 * cc + K * 4, mac=3 * 64 * K * V + 2 * 64 * 64 * V)
    m["kda_intra"] = dict(bytes=2 * qk + f32 + 3 * cc + 3 * f32 + K * 4 + 3 * f32 + 64 * 4,
                          mac=2 * 64 ** 3 + 4 * 64 * 64 * K)
    return m


class ClockSampler:
    """``nvidia-smi`` clocks and throttle reasons, sampled every 200 ms while the timed region runs."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.proc = index, None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                                          "-lms", "200", "-i", str(self.index)], stdout=subprocess.PIPE, text=True)
        except OSError:
            self.proc = None
        return self

    def __exit__(self, *exc):
        self.samples = []
        if self.proc is None:
            return
        time.sleep(0.25)
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        for line in out.splitlines():
            parts = [x.strip() for x in line.split(",")]
            if len(parts) >= 9:
                self.samples.append(parts)

    def summary(self) -> dict:
        if not getattr(self, "samples", None):
            return dict(sm_mhz=None, sm_max_mhz=None, reasons=["unsampled"])
        sm = [float(s[1]) for s in self.samples if s[1].replace(".", "").isdigit()]
        mx = [float(s[2]) for s in self.samples if s[2].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({n for s in self.samples for n, v in zip(names, s[5:9]) if v.lower().startswith("active")})
        return dict(sm_mhz=statistics.median(sm) if sm else None, sm_max_mhz=max(mx) if mx else None, reasons=reasons,
                    samples=len(self.samples))


def host_case(workload: str, seed: int) -> dict:
    from oracle.cases import baseline_config

    return baseline_config(WORKLOADS[workload]["index"], seed=seed)


def longctx_device_inputs(device, rank: int, world: int, seed: int = 0) -> dict:
    """Config 4 shard of this rank, drawn on the device (17 GB of fp32 NumPy per tensor would not fit a host
    round trip): q, k ~ N(0,1) L2-normalised, v, dO ~ N(0,1), beta = sigmoid(N(0,1)), g = logsigmoid(N(0,1)+3);
    document lengths U[4096, 131072] drawn once on the host for the whole sequence."""
    from oracle.cases import uniform_docs

    tl = LONG_T // world
    gen = torch.Generator(device=device).manual_seed(seed * 1000 + rank)

    def randn(*shape):
        return torch.randn(*shape, generator=gen, device=device, dtype=torch.float32)

    def unit(x):
        return (x * torch.rsqrt((x * x).sum(-1, keepdim=True) + 1e-6)).to(torch.bfloat16)

    seg = torch.from_numpy(uniform_docs(np.random.default_rng(seed), 1, LONG_T, 4096, 131072))
    out = dict(q=unit(randn(1, tl, 16, 128)), k=unit(randn(1, tl, 16, 128)), v=randn(1, tl, 16, 128).to(torch.bfloat16),
               do=randn(1, tl, 16, 128).to(torch.bfloat16), beta=torch.sigmoid(randn(1, tl, 16)),
               g=torch.nn.functional.logsigmoid(randn(1, tl, 16) + 3.0))
    out["seg"] = seg[:, rank * tl:(rank + 1) * tl].to(device=device, dtype=torch.int32)
    if world == 1:
        ids = out["seg"][0]
        starts = torch.nonzero(ids[1:] != ids[:-1]).flatten() + 1
        out["cu"] = torch.cat([starts.new_zeros(1), starts, starts.new_full((1,), ids.numel())]).to(torch.int32)
    return out


def to_torch_host(case: dict, workload: str) -> dict:
    """Pinned host tensors in the dtypes of the op call."""
    out = {}
    half = ("q", "k", "v", "do") if workload != "ssd" else ("x", "B", "C", "do")
    for name, arr in case.items():
        if name == "meta" or name in ("h0", "dht"):
            continue
        t = torch.from_numpy(np.ascontiguousarray(arr))
        if name in half:
            t = t.to(torch.bfloat16)
        elif name == "seg":
            t = t.to(torch.int32)
        else:
            t = t.to(torch.float32)
        out[name] = t.pin_memory() if torch.cuda.is_available() else t
    return out


GRAD_NAMES = {"gdn": ("q", "k", "v", "g", "beta"), "kda": ("q", "k", "v", "g", "beta"),
              "ssd": ("x", "dt", "A", "B", "C"), "longctx": ("q", "k", "v", "g", "beta")}


def run_step(workload: str, dev: dict):
    """One forward + backward through the public API on device tensors; returns (o, grads)."""
    from jax_linear_attention_b200 import ops

    names = GRAD_NAMES[workload]
    leaves = [dev[n].requires_grad_(True) for n in names]
    if workload == "ssd":
        from jax_linear_attention_b200.layers.ssm import mamba2_ssd

        o, _ = mamba2_ssd(dev["x"], dev["dt"], dev["A"], dev["B"], dev["C"], d=dev["D"], segment_ids=dev.get("seg"))
    elif workload == "longctx":
        if "cu" in dev:  # one GPU: the documents are the rows
            o, _ = ops.linear_attention("gated_deltanet", dev["q"], dev["k"], dev["v"], g=dev["g"], beta=dev["beta"],
                                        cu_seqlens=dev["cu"])
        else:
            from jax_linear_attention_b200.distributed import context_parallel_linear_attention

            # documents (4 Ki .. 128 Ki tokens) are cut into pieces of 8192 tokens (128 chunks: 16 pieces x 16 heads per
            # rank at 8 GPUs) so that the state passes fill the SMs instead of walking each document as one chain;
            # shorter pieces only lengthen the scan over the pieces (measured at 8 GPUs: 16 / 24 / 32 / 64 / 96 pieces
            # per rank -> 9.2 / 9.4 / 9.7 / 11.1 / 11.5 ms)
            if "plan" not in dev:  # the document layout is fixed input metadata: cut it into pieces once
                from jax_linear_attention_b200.distributed import plan_pieces

                dev["plan"] = plan_pieces(dev["seg"], 8192)
            o, _ = context_parallel_linear_attention("gated_deltanet", dev["q"], dev["k"], dev["v"], g=dev["g"],
                                                     beta=dev["beta"], segment_ids=dev["seg"], piece_len=dev["plan"])
    else:
        kind = "gated_deltanet" if workload == "gdn" else "kda"
        o, _ = ops.linear_attention(kind, dev["q"], dev["k"], dev["v"], g=dev["g"], beta=dev["beta"],
                                    segment_ids=dev.get("seg"))
    grads = torch.autograd.grad(o, leaves, dev["do"])
    return o, grads


def profile_table(lib) -> dict:
    lib.jla_profile_kernel_name.restype = C.c_char_p
    out = {}
    i = 0
    while True:
        name = lib.jla_profile_kernel_name(i)
        if name is None:
            break
        ms, n = C.c_double(0), C.c_int(0)
        lib.jla_profile_read(i, C.byref(ms), C.byref(n))
        if n.value:
            out[name.decode()] = dict(launches=n.value, total_ms=ms.value)
        i += 1
    return out


def cpu_port_step(case: dict, rows: int) -> float:
    """Seconds for one fwd+bwd of the oracle's chunk-64 algorithm (float32, autograd) on the first `rows` batch
    rows of the case."""
    from oracle import chunked as oc

    f32 = torch.float32
    names = ("q", "k", "v", "g", "beta")
    t = {n: torch.tensor(case[n][:rows], dtype=f32, requires_grad=True) for n in names}
    seg = torch.tensor(case["seg"][:rows]) if "seg" in case else None
    do = torch.tensor(case["do"][:rows], dtype=f32)
    t0 = time.perf_counter()
    fn = oc.gated_delta_rule if t["g"].ndim == 3 else oc.kda
    o, _ = fn(t["q"], t["k"], t["v"], t["g"], t["beta"], segment_ids=seg, dtype=f32)
    torch.autograd.grad(o, [t[n] for n in names], do)
    return time.perf_counter() - t0


def cpu_baseline(case: dict, rows: int = 1, budget_s: float = 12.0) -> dict:
    """The oracle port timed on a bounded sample: ``rows`` batch rows per pass, passes repeated until about
    ``budget_s`` seconds of CPU work are spent (one untimed pass first)."""
    cpu_port_step(case, rows)
    times = []
    while sum(times) < budget_s and len(times) < 64:
        times.append(cpu_port_step(case, rows))
    T = case["q"].shape[1]
    mean = sum(times) / len(times)
    return dict(value=rows * T / mean, unit="tokens/s", cores=torch.get_num_threads(), kind="port",
                sample=f"{rows} of {case['q'].shape[0]} batch rows (T={T}, all heads), fwd+bwd via autograd of the "
                       f"chunk-64 oracle in float32; mean of {len(times)} passes, {sum(times):.1f} s in all")


def run_reference(args) -> None:
    """The reference arm: the CPU port of the reference's chunked algorithm on this host's cores."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    case = host_case(args.workload, seed=0)
    rows = 1
    for _ in range(max(args.warmup, 0) and 1):
        cpu_port_step(case, rows)
    steps = max(1, min(args.steps, 3))
    t0 = time.perf_counter()
    for _ in range(steps):
        cpu_port_step(case, rows)
    dt = (time.perf_counter() - t0) / steps
    T = case["q"].shape[1]
    value = rows * T / dt
    sample = (f"each step = fwd+bwd of {rows} of {case['q'].shape[0]} batch rows (T={T}, all heads) with the chunk-64 "
              f"oracle port in float32 on {torch.get_num_threads()} threads; {steps} timed steps")
    line = dict(impl="reference", metric=METRIC, value=value, unit="tokens/s", n_gpus=args.gpus, steps=steps,
                warmup=1 if args.warmup else 0, ms_per_step=dt * 1e3, higher_is_better=True, scaling="weak",
                vs_baseline=None, dtype="f32", data="synthetic",
                config=dict(workload=WORKLOADS[args.workload]["name"], note="CPU port of src/jla/ops/chunked.py; the "
                            "reference's JAX CPU path is unavailable on this box (JAX not installed)"),
                cpu_baseline=dict(value=value, unit="tokens/s", cores=torch.get_num_threads(), kind="port", sample=sample),
                e2e=dict(value=value, unit="tokens/s", h2d_bytes_per_step=0, d2h_bytes_per_step=0))
    print(json.dumps(line))


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="gdn", choices=sorted(WORKLOADS))
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer pass (for profiler captures)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    if args.impl == "reference":
        run_reference(args)
        return

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the CUDA kernels have no CPU fallback")
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    dist = None
    if world > 1:
        import torch.distributed as dist

        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=device)

    from jax_linear_attention_b200 import _lib

    lib = _lib.load()
    longctx = args.workload == "longctx"
    if longctx:
        dev = longctx_device_inputs(device, rank, world)
        host = {n: t.cpu().pin_memory() for n, t in dev.items() if n != "cu"}
        case = {"q": dev["q"], "v": dev["v"]}
        shape = (1, LONG_T // world)
        tokens = LONG_T // world  # per rank; the job processes LONG_T tokens per step (strong scaling)
        args.steps = min(args.steps, 5)
    else:
        case = host_case(args.workload, seed=rank)
        host = to_torch_host(case, args.workload)
        dev = {n: t.to(device, non_blocking=True) for n, t in host.items()}
        shape = case["q"].shape if "q" in case else case["x"].shape
        tokens = shape[0] * shape[1]
    torch.cuda.synchronize()

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- device-resident timing
    for _ in range(args.warmup):
        run_step(args.workload, dev)
    lib.jla_profile_enable(1)
    lib.jla_profile_reset()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(local) as clocks:
        e0.record()
        for _ in range(args.steps):
            run_step(args.workload, dev)
        e1.record()
        barrier()
    ms = e0.elapsed_time(e1)
    prof = profile_table(lib)
    lib.jla_profile_enable(0)
    if dist is not None:
        tms = torch.tensor([ms], device=device)
        dist.all_reduce(tms, op=dist.ReduceOp.MAX)
        ms = float(tms.item())
    ms_per_step = ms / args.steps

    # ---- end to end: pinned host inputs -> device -> fwd+bwd -> results back to pinned host memory
    out_host = None
    h2d = sum(t.numel() * t.element_size() for t in host.values())

    # Three streams: step i+1's inputs cross PCIe while step i computes and step i-1's results go back, as a
    # training or serving loop feeding this op from host memory would run it. Every step still copies all of its
    # inputs in and all of its results out inside the timed region.
    s_in, s_out = torch.cuda.Stream(device), torch.cuda.Stream(device)

    def e2e_step():
        nonlocal out_host
        cur = torch.cuda.current_stream(device)
        with torch.cuda.stream(s_in):
            d = {n: t.to(device, non_blocking=True) for n, t in host.items()}
            ready = torch.cuda.Event()
            ready.record(s_in)
        cur.wait_event(ready)
        for t in d.values():
            t.record_stream(cur)
        if "cu" in dev:
            d["cu"] = dev["cu"]
        o, grads = run_step(args.workload, d)
        outs = [o.detach(), *grads]
        done = torch.cuda.Event()
        done.record(cur)
        if out_host is None:
            out_host = [torch.empty(x.shape, dtype=x.dtype).pin_memory() for x in outs]
        with torch.cuda.stream(s_out):
            s_out.wait_event(done)
            for dst, src in zip(out_host, outs):
                dst.copy_(src, non_blocking=True)
                src.record_stream(s_out)

    e2e_steps = 0 if args.no_e2e else max(3, min(args.steps, 10))
    for _ in range(4 if e2e_steps else 0):  # untimed: the caching allocator reaches its steady state on all three streams
        e2e_step()
    barrier()
    e0.record()
    for _ in range(e2e_steps):
        e2e_step()
    torch.cuda.current_stream(device).wait_stream(s_out)
    e1.record()
    barrier()
    e2e_ms = e0.elapsed_time(e1)
    if dist is not None:
        tms = torch.tensor([e2e_ms], device=device)
        dist.all_reduce(tms, op=dist.ReduceOp.MAX)
        e2e_ms = float(tms.item())
    d2h = sum(t.numel() * t.element_size() for t in out_host) if out_host else 0

    if rank == 0:
        pk = peaks()
        launches = sum(v["launches"] for v in prof.values())
        K, V = (case["q"].shape[3], case["v"].shape[3]) if "q" in case else (case["B"].shape[3], case["x"].shape[3])
        H = case["v"].shape[2] if "v" in case else case["x"].shape[2]
        units = (tokens // CHUNK) * H  # (chunk, head) pairs per launch
        model = kernel_model(K, V, delta=args.workload != "ssd", save=True)
        roof = None
        if prof:
            top = max(prof, key=lambda n: prof[n]["total_ms"])
            per_launch_ms = prof[top]["total_ms"] / prof[top]["launches"]
            if top in model:
                by = model[top]["bytes"] * units
                fl = 2 * model[top]["mac"] * units
                t_hbm = by / (pk["hbm_gbs"] * 1e9)
                t_tc = fl / (pk["bf16_tflops"] * 1e12)
                if t_hbm >= t_tc:
                    ach = by / (per_launch_ms * 1e-3) / 1e9
                    roof = dict(bound="hbm", achieved=ach, peak=pk["hbm_gbs"], unit="GB/s", frac=ach / pk["hbm_gbs"])
                else:
                    ach = fl / (per_launch_ms * 1e-3) / 1e12
                    roof = dict(bound="tensor", achieved=ach, peak=pk["bf16_tflops"], unit="TFLOP/s",
                                frac=ach / pk["bf16_tflops"])
                # DRAM bytes per unit from ncu captures of this workload (profiles/*.md); scaled by the units of a launch
                ncu_bytes_per_unit = {"sg_grads_k": 805.7e6 / 4096, "sg_grads_q": 491.2e6 / 4096,
                                      "sg_bwd_state": 454.0e6 / 4096, "kkt_inv": 92.9e6 / 4096}
                ncu_kda = {"kda_intra": 1023.5e6 / 4208, "kda_prep": 524.4e6 / 4208, "kda_chunk_grads": 1038.4e6 / 4208}
                traffic = (ncu_bytes_per_unit.get(top) if args.workload == "gdn"
                           else ncu_kda.get(top) if args.workload == "kda" else None)
                roof.update(kernel=top, ms_per_launch=per_launch_ms,
                            traffic=None if traffic is None else traffic * units, peak_source=pk["source"],
                            algorithmic_bytes_per_launch=by, algorithmic_flops_per_launch=fl)
        # whole-step view against both rooflines (dense 64x64 tiles, no recompute, inverse excluded: 491,520 FLOP and
        # 2,816 B per token and head for the delta-rule kinds)
        step_flops = 491520.0 * tokens * H if args.workload != "ssd" else 172032.0 * tokens * H
        step_bytes = 2816.0 * tokens * H
        sec = ms_per_step * 1e-3
        line = dict(
            metric=METRICS[args.workload] or METRIC, value=world * tokens / sec, unit="tokens/s", n_gpus=world,
            steps=args.steps, warmup=args.warmup, ms_per_step=ms_per_step, higher_is_better=True,
            scaling="strong" if longctx else "weak", vs_baseline=None,
            dtype="bf16", data="synthetic",
            config=dict(workload=WORKLOADS[args.workload]["name"], per_gpu_batch=list(shape[:2]),
                        l2="inputs larger than L2 (hundreds of MB of q,k,v,dO + residuals per step)",
                        parallelism=(f"sequence-parallel over {world} GPUs: documents cut into pieces joined by affine "
                                     "maps, NCCL send/recv of the fp32 state" if longctx and world > 1
                                     else "one GPU, documents as cu_seqlens rows" if longctx
                                     else f"batch x heads, {world} GPU(s), no communication")),
            e2e=None if not e2e_steps else dict(
                value=world * tokens / (e2e_ms / e2e_steps * 1e-3), unit="tokens/s", h2d_bytes_per_step=h2d,
                d2h_bytes_per_step=d2h, steps=e2e_steps, ms_per_step=e2e_ms / e2e_steps),
            gpu_launches=launches,
            clocks=clocks.summary(),
            roofline=roof,
            step=dict(tflops_algorithmic=step_flops / sec / 1e12, frac_of_bf16_peak=step_flops / sec / 1e12 / pk["bf16_tflops"],
                      gbs_algorithmic=step_bytes / sec / 1e9, frac_of_hbm_peak=step_bytes / sec / 1e9 / pk["hbm_gbs"]),
            kernels={n: dict(launches=v["launches"], ms_per_launch=v["total_ms"] / v["launches"]) for n, v in prof.items()},
        )
        if not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_baseline(case, rows=4) if args.workload in ("gdn", "kda") else None
        print(json.dumps(line))
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
