"""Benchmark of the hot path: Gated DeltaNet chunk forward + backward at B8 T2048 H16 K = V = 128, bf16, packed documents.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload gdn|ssd|kda|gdn2|gdnv256|longctx]

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

Timing: a block is exactly ``--steps`` steps between two CUDA events, bracketed by a barrier and a device
synchronisation, maximum over the ranks. Blocks are repeated until a second of GPU time has been spent;
``ms_per_step`` and ``value`` are the median block, ``blocks`` lists the spread.

With N > 1 two more curves are measured after the headline and reported under extra keys of the same line:
``strong`` (the same B8 T2048 H16 problem cut over the N ranks by batch x heads through ``shard_kernel_call``)
and ``longctx`` (one 1,064,960-token sequence cut over the N ranks along T, NCCL send/recv of the fp32 state),
each with a correctness check of one shard against an unsharded run.
"""

from __future__ import annotations

import argparse
import ctypes as C
import hashlib
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

import numpy as np  # noqa: E402
import torch  # noqa: E402

METRIC = "GDN chunk fwd+bwd tokens/s/GPU (B8·T2048·H16·d128 bf16); % bf16 TC peak"
CHUNK = 64

WORKLOADS = {
    "gdn": dict(name="config1: gated_deltanet B8 T2048 H16 K128 V128 chunk64 bf16, packed docs U[64,2048]", index=1),
    "ssd": dict(name="config2: mamba2 SSD B8 T2048 H64 P64 N128 G1 bf16", index=2),
    "kda": dict(name="config3: kda B4 T4096 H16 K128 V128 bf16, packed docs U[128,4096]", index=3),
    "gdn2": dict(name="gdn2 (Gated DeltaNet-2, erase and write gates per channel) at config3's shape: B4 T4096 H16 K128 "
                      "V128 bf16, packed docs U[128,4096]", index=None),
    "gdnv256": dict(name="gated_deltanet with wide value heads (head 128, expand_v = 2): B8 T2048 H16 K128 V256 bf16, "
                         "packed docs U[64,2048]; the chunk kernels run each head as two blocks of 128 value channels",
                    index=None),
    "longctx": dict(name="config4: gated_deltanet B1 T1064960 H16 K128 V128 bf16, packed docs U[4096,131072], "
                         "sequence-parallel over the ranks", index=4),
}
METRICS = {
    "gdn": None,  # the headline metric
    "ssd": "Mamba-2 SSD chunk fwd+bwd tokens/s (B8·T2048·H64·P64·N128 bf16)",
    "kda": "KDA fwd+bwd tokens/s (B4·T4096·H16·d128 bf16)",
    "gdn2": "Gated DeltaNet-2 fwd+bwd tokens/s (B4·T4096·H16·d128 bf16)",
    "gdnv256": "GDN fwd+bwd tokens/s with wide value heads (B8·T2048·H16·K128·V256 bf16)",
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
    from oracle.cases import baseline_config, make_case

    if workload == "gdn2":  # no published configuration: the KDA workload's shape and gates, b and w as sigmoids
        return make_case("gdn2", seed=seed, B=4, T=4096, H=16, K=128, V=128, dtype="bfloat16", gates="kda_baseline",
                         docs="uniform", doc_range=(128, 4096))
    if workload == "gdnv256":  # config 1's batch, documents and gates with twice the value channels per head
        return make_case("gated_deltanet", seed=seed, B=8, T=2048, H=16, K=128, V=256, dtype="bfloat16",
                         gates="baseline", docs="uniform", doc_range=(64, 2048))
    return baseline_config(WORKLOADS[workload]["index"], seed=seed)


LONG_BLOCKS = 32  # the long sequence is drawn in 32 blocks of 33,280 tokens, each from its own seed, so that any
                  # rank of 1, 2, 4 or 8 draws exactly its tokens and every world size sees the same sequence


def longctx_device_inputs(device, rank: int, world: int, seed: int = 0) -> dict:
    """The 1,064,960-token workload's shard of this rank, drawn on the device (17 GB of fp32 NumPy per tensor would
    not fit a host round trip): q, k ~ N(0,1) L2-normalised, v, dO ~ N(0,1), beta = sigmoid(N(0,1)),
    g = logsigmoid(N(0,1)+3); document lengths U[4096, 131072] drawn once on the host for the whole sequence."""
    from oracle.cases import uniform_docs

    tl = LONG_T // world
    tb = LONG_T // LONG_BLOCKS
    per = LONG_BLOCKS // world

    def unit(x):
        return (x * torch.rsqrt((x * x).sum(-1, keepdim=True) + 1e-6)).to(torch.bfloat16)

    parts = {n: [] for n in ("q", "k", "v", "do", "beta", "g")}
    for blk in range(rank * per, (rank + 1) * per):
        gen = torch.Generator(device=device).manual_seed(seed * 1000 + blk)

        def randn(*shape):
            return torch.randn(*shape, generator=gen, device=device, dtype=torch.float32)

        parts["q"].append(unit(randn(1, tb, 16, 128)))
        parts["k"].append(unit(randn(1, tb, 16, 128)))
        parts["v"].append(randn(1, tb, 16, 128).to(torch.bfloat16))
        parts["do"].append(randn(1, tb, 16, 128).to(torch.bfloat16))
        parts["beta"].append(torch.sigmoid(randn(1, tb, 16)))
        parts["g"].append(torch.nn.functional.logsigmoid(randn(1, tb, 16) + 3.0))
    out = {n: torch.cat(v, dim=1) if len(v) > 1 else v[0] for n, v in parts.items()}
    seg = torch.from_numpy(uniform_docs(np.random.default_rng(seed), 1, LONG_T, 4096, 131072))
    out["seg"] = seg[:, rank * tl:(rank + 1) * tl].to(device=device, dtype=torch.int32)
    if world == 1:
        ids = out["seg"][0]
        starts = torch.nonzero(ids[1:] != ids[:-1]).flatten() + 1
        out["cu"] = torch.cat([starts.new_zeros(1), starts, starts.new_full((1,), ids.numel())]).to(torch.int32)
    return out


def to_torch_host(case: dict, workload: str) -> dict:
    """Pinned host tensors in the dtypes of the op call."""
    out = {}
    half = ("q", "k", "v", "do", "b", "w") if workload != "ssd" else ("x", "B", "C", "do")
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
              "gdn2": ("q", "k", "v", "g", "b", "w"), "gdnv256": ("q", "k", "v", "g", "beta"),
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
    elif workload == "gdn2":
        o, _ = ops.linear_attention("gdn2", dev["q"], dev["k"], dev["v"], g=dev["g"], b=dev["b"], w=dev["w"],
                                    segment_ids=dev.get("seg"))
    else:
        kind = "kda" if workload == "kda" else "gated_deltanet"
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


CPU_ROWS = 4  # batch rows of the workload that one CPU pass computes (both CPU legs use the same sample)


def cpu_baseline(case: dict, rows: int = CPU_ROWS, budget_s: float = 12.0) -> dict:
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
    """The reference arm: the CPU port of the reference's chunked algorithm on this host's cores. One step is one
    fwd+bwd over the same bounded sample the ``cpu_baseline`` leg uses; ``--steps`` and ``--warmup`` are honoured up
    to 50 steps (a step takes about a second)."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    if args.workload not in ("gdn", "kda"):
        emit_line(dict(impl="reference", unavailable=f"the timed CPU port covers the gdn and kda workloads, not "
                                                      f"{args.workload}"))
        return
    case = host_case(args.workload, seed=0)
    rows = min(CPU_ROWS, case["q"].shape[0])
    warmup = max(0, min(args.warmup, 5))
    for _ in range(warmup):
        cpu_port_step(case, rows)
    steps = max(1, min(args.steps, 50))
    t0 = time.perf_counter()
    for _ in range(steps):
        cpu_port_step(case, rows)
    dt = (time.perf_counter() - t0) / steps
    T = case["q"].shape[1]
    value = rows * T / dt
    sample = (f"each step = fwd+bwd of {rows} of {case['q'].shape[0]} batch rows (T={T}, all heads) with the chunk-64 "
              f"oracle port in float32 on {torch.get_num_threads()} threads; {steps} timed steps")
    line = dict(impl="reference", metric=METRIC, value=value, unit="tokens/s", n_gpus=args.gpus, steps=steps,
                warmup=warmup, ms_per_step=dt * 1e3, higher_is_better=True, scaling="weak",
                vs_baseline=None, dtype="f32", data="synthetic",
                config=dict(workload=WORKLOADS[args.workload]["name"], note="CPU port of src/jla/ops/chunked.py; the "
                            "reference's JAX CPU path is unavailable on this box (JAX not installed)"),
                cpu_baseline=dict(value=value, unit="tokens/s", cores=torch.get_num_threads(), kind="port", sample=sample),
                e2e=dict(value=value, unit="tokens/s", h2d_bytes_per_step=0, d2h_bytes_per_step=0))
    emit_line(line)


def bind_to_gpu_numa_node(local: int) -> str:
    """Pins this process to the CPUs next to its GPU (read from sysfs) before any pinned buffer is allocated, so that
    the host side of every PCIe copy is local memory. Host-side scheduling only; returns what was done."""
    try:
        props = torch.cuda.get_device_properties(local)
        bdf = f"{props.pci_domain_id:04x}:{props.pci_bus_id:02x}:{props.pci_device_id:02x}.0"
        with open(f"/sys/bus/pci/devices/{bdf}/local_cpulist") as f:
            text = f.read().strip()
        cpus = set()
        for part in text.split(","):
            lo, _, hi = part.partition("-")
            cpus.update(range(int(lo), int(hi or lo) + 1))
        cpus &= os.sched_getaffinity(0)
        if not cpus:
            return f"{bdf}: no usable CPU in {text}"
        os.sched_setaffinity(0, cpus)
        return f"{bdf}: {len(cpus)} CPUs ({text})"
    except (OSError, AttributeError, ValueError) as err:
        return f"not bound ({type(err).__name__}: {err})"


TRAFFIC_FILE = os.path.join(ROOT, "profiles", "dram_traffic.json")


def profiled_traffic(kernel: str, workload: str):
    """DRAM bytes per (chunk, head) unit of ``kernel`` from a committed ncu capture, or None when there is none or the
    kernel's source changed after the capture (the file keeps a hash of the source next to each figure)."""
    try:
        with open(TRAFFIC_FILE) as f:
            table = json.load(f)
    except (OSError, ValueError):
        return None
    entry = table.get(workload, {}).get(kernel)
    if not entry:
        return None
    try:
        with open(os.path.join(ROOT, entry["source"]), "rb") as f:
            digest = hashlib.sha256(f.read()).hexdigest()[:16]
    except OSError:
        return None
    if digest != entry.get("source_sha256_16"):
        return None
    return dict(bytes_per_unit=entry["dram_bytes"] / entry["units"], commit=entry.get("commit"))


class Deadline:
    """Extras measured after the headline must never cost the headline: if they have not finished ``seconds`` after
    they began, rank 0 prints the line as it stands and every rank leaves."""

    def __init__(self, seconds: float, on_expire):
        self.timer = threading.Timer(seconds, on_expire)
        self.timer.daemon = True

    def __enter__(self):
        self.timer.start()
        return self

    def __exit__(self, *exc):
        self.timer.cancel()


_LINE_FD = None  # the process's original standard output once main() has claimed it


def claim_stdout() -> None:
    """The contract is ONE JSON line on standard output. Libraries write there too (NCCL prints its version line on
    file descriptor 1 when the first communicator comes up), so descriptor 1 is pointed at standard error for the
    whole run and the line goes to a saved copy of the original."""
    global _LINE_FD
    sys.stdout.flush()
    _LINE_FD = os.dup(1)
    os.dup2(2, 1)


def emit_line(line: dict) -> None:
    text = (json.dumps(line) + "\n").encode()
    if _LINE_FD is None:
        sys.stdout.write(text.decode())
        sys.stdout.flush()
    else:
        os.write(_LINE_FD, text)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="gdn", choices=sorted(WORKLOADS))
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer pass (for profiler captures)")
    ap.add_argument("--no-extras", action="store_true", help="N > 1: skip the strong-scaling and long-context curves")
    ap.add_argument("--single-block", action="store_true", help="time one block of --steps steps only (profiler captures)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    claim_stdout()
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
    numa = bind_to_gpu_numa_node(local)
    dist = None
    if world > 1:
        import torch.distributed as dist

        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=device)
        every = [None] * world
        dist.all_gather_object(every, numa)
        numa = every  # one entry per rank

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

    def max_over_ranks(ms: float) -> float:
        if dist is None:
            return ms
        tms = torch.tensor([ms], device=device)
        dist.all_reduce(tms, op=dist.ReduceOp.MAX)
        return float(tms.item())

    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)

    def timed_block(step_fn, steps: int) -> float:
        """Exactly ``steps`` steps between two events, barrier + synchronise on both sides; ms, max over ranks."""
        barrier()
        e0.record()
        for _ in range(steps):
            step_fn()
        e1.record()
        barrier()
        return max_over_ranks(e0.elapsed_time(e1))

    # ---- device-resident timing
    for _ in range(args.warmup):
        run_step(args.workload, dev)
    # Blocks alternate: one without the library's per-kernel events (the headline: two event records around every
    # kernel cost about 4 % of a step), one with them (the per-kernel times of the roofline), until the headline
    # blocks add up to a second.
    lib.jla_profile_enable(1)
    lib.jla_profile_reset()
    blocks_ms, prof_blocks_ms = [], []
    with ClockSampler(local) as clocks:
        while True:
            if not args.single_block:
                lib.jla_profile_enable(0)
                blocks_ms.append(timed_block(lambda: run_step(args.workload, dev), args.steps))
                lib.jla_profile_enable(1)
            prof_blocks_ms.append(timed_block(lambda: run_step(args.workload, dev), args.steps))
            if args.single_block or sum(blocks_ms) >= 1000.0 or len(blocks_ms) >= 400:
                break
    prof = profile_table(lib)
    lib.jla_profile_enable(0)
    if not blocks_ms:
        blocks_ms = prof_blocks_ms
    ms = statistics.median(blocks_ms)
    ms_per_step = ms / args.steps
    status_after_timing = _lib.device_status()

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

    e2e_steps = 0 if args.no_e2e else max(3, min(args.steps, 40))  # (the pipeline's fill and drain are inside the region)
    for _ in range(4 if e2e_steps else 0):  # untimed: the caching allocator reaches its steady state on all three streams
        e2e_step()
    barrier()
    e0.record()
    for _ in range(e2e_steps):
        e2e_step()
    torch.cuda.current_stream(device).wait_stream(s_out)
    e1.record()
    barrier()
    e2e_ms = max_over_ranks(e0.elapsed_time(e1))
    d2h = sum(t.numel() * t.element_size() for t in out_host) if out_host else 0

    line = None
    if rank == 0:
        pk = peaks()
        launches = sum(v["launches"] for v in prof.values()) // max(len(prof_blocks_ms), 1)  # per timed block
        K, V = (case["q"].shape[3], case["v"].shape[3]) if "q" in case else (case["B"].shape[3], case["x"].shape[3])
        H = case["v"].shape[2] if "v" in case else case["x"].shape[2]
        if V > 128 and V % 128 == 0:  # wide value heads run as V / 128 heads of 128 channels: count those
            H, V = H * (V // 128), 128
        units = (tokens // CHUNK) * H  # (chunk, head) pairs per launch
        model = kernel_model(K, V, delta=args.workload != "ssd", save=True)
        roof = None
        step_traffic = 0.0
        step_traffic_known = bool(prof)
        for name in prof:  # DRAM bytes of the whole step from the committed captures, if every kernel has a current one
            t = profiled_traffic(name, args.workload)
            small = prof[name]["total_ms"] / prof[name]["launches"] < 0.03  # table and gate prologues: a few MB
            if t is None and not small:
                step_traffic_known = False
            elif t is not None:  # (a kernel may launch more than once per step: the two key-gradient finalisers)
                step_traffic += t["bytes_per_unit"] * units * prof[name]["launches"] / (len(prof_blocks_ms) * args.steps)
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
                t = profiled_traffic(top, args.workload)
                roof.update(kernel=top, ms_per_launch=per_launch_ms,
                            traffic=None if t is None else t["bytes_per_unit"] * units,
                            traffic_measured_at=None if t is None else t["commit"], peak_source=pk["source"],
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
                        timing=f"median of {len(blocks_ms)} blocks of {args.steps} steps (CUDA events, barrier + "
                               "synchronise around each block, max over ranks); per-kernel times from as many "
                               "interleaved blocks with the library's events around every kernel",
                        host_binding=numa,
                        parallelism=(f"sequence-parallel over {world} GPUs: documents cut into pieces joined by affine "
                                     "maps, NCCL send/recv of the fp32 state" if longctx and world > 1
                                     else "one GPU, documents as cu_seqlens rows" if longctx
                                     else f"batch x heads, {world} GPU(s), no communication")),
            blocks=dict(count=len(blocks_ms), ms_per_step_median=ms_per_step, ms_per_step_min=min(blocks_ms) / args.steps,
                        ms_per_step_max=max(blocks_ms) / args.steps, ms_per_step_first=blocks_ms[0] / args.steps,
                        total_timed_ms=sum(blocks_ms),
                        ms_per_step_median_with_kernel_events=statistics.median(prof_blocks_ms) / args.steps),
            e2e=None if not e2e_steps else dict(
                value=world * tokens / (e2e_ms / e2e_steps * 1e-3), unit="tokens/s", h2d_bytes_per_step=h2d,
                d2h_bytes_per_step=d2h, steps=e2e_steps, ms_per_step=e2e_ms / e2e_steps),
            gpu_launches=launches,
            device_status=status_after_timing,
            clocks=clocks.summary(),
            roofline=roof,
            step=dict(tflops_algorithmic=step_flops / sec / 1e12, frac_of_bf16_peak=step_flops / sec / 1e12 / pk["bf16_tflops"],
                      gbs_algorithmic=step_bytes / sec / 1e9, frac_of_hbm_peak=step_bytes / sec / 1e9 / pk["hbm_gbs"],
                      min_traffic_bytes=step_bytes,
                      step_traffic_bytes=step_traffic if step_traffic_known else None,
                      traffic_over_minimum=step_traffic / step_bytes if step_traffic_known else None),
            kernels={n: dict(launches=v["launches"], ms_per_launch=v["total_ms"] / v["launches"]) for n, v in prof.items()},
        )
        if not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_baseline(case) if args.workload in ("gdn", "kda") else None

    # ---- N > 1: the curves that the weak-scaling headline cannot show
    if world > 1 and args.workload == "gdn" and not args.no_extras:
        printed = threading.Event()

        def emit():
            if rank == 0 and not printed.is_set():
                printed.set()
                emit_line(line)

        def expire():
            if rank == 0:
                for key in ("strong", "longctx"):
                    line.setdefault(key, dict(error="not finished within the time limit of the extra measurements"))
            emit()
            os._exit(0)

        with Deadline(240.0, expire):
            for key, fn in (("strong", strong_scaling), ("longctx", longctx_curve)):
                try:
                    res = fn(device, rank, world, dist, timed_block, ms_per_step, dev)
                except Exception as err:  # an extra must not cost the headline
                    res = dict(error=f"{type(err).__name__}: {err}"[:300])
                if rank == 0:
                    line[key] = res
        emit()
    elif rank == 0:
        emit_line(line)
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


def strong_scaling(device, rank, world, dist, timed_block, one_gpu_ms_per_step, rank0_dev) -> dict:
    """The B8 T2048 H16 d128 problem of seed 0 cut over the ranks by batch x heads (``shard_kernel_call``: batch
    first, then heads; no collective). Rank 0's weak-scaling problem is that very problem, so its unsharded output
    and time are the references: the shard must equal the matching slice bit for bit."""
    from jax_linear_attention_b200 import ops
    from jax_linear_attention_b200.distributed import plan_shards, shard_kernel_call, shard_slices

    case = host_case("gdn", seed=0)
    t = {n: torch.from_numpy(np.ascontiguousarray(case[n])) for n in ("q", "k", "v", "g", "beta", "do", "seg")}
    B, T, H = case["v"].shape[:3]
    bs, hs, ks = shard_slices(plan_shards(B, H, H, world), rank, B, H, H)
    half = ("q", "k", "v", "do")
    full = {n: (x.to(torch.bfloat16) if n in half else x.to(torch.int32) if n == "seg" else x.float()) for n, x in t.items()}
    # every rank keeps only its shard on the device; shard_kernel_call slices the (here already local) tensors
    loc = dict(q=full["q"][bs][:, :, ks], k=full["k"][bs][:, :, ks], v=full["v"][bs][:, :, hs], g=full["g"][bs][:, :, hs],
               beta=full["beta"][bs][:, :, hs], do=full["do"][bs][:, :, hs], seg=full["seg"][bs])
    loc = {n: x.contiguous().to(device) for n, x in loc.items()}

    def fn(q, k, v, g, beta, **opts):
        return ops.linear_attention("gated_deltanet", q, k, v, g=g, beta=beta, **opts)

    def step():
        leaves = [loc[n].requires_grad_(True) for n in ("q", "k", "v", "g", "beta")]
        o, _ = shard_kernel_call(fn, leaves[0], leaves[1], leaves[2], leaves[3:], dict(segment_ids=loc["seg"]),
                                 rank=0, world=1, supports=ops.cuda.SUPPORTS["gated_deltanet"])
        return o, torch.autograd.grad(o, leaves, loc["do"])

    for _ in range(3):
        o, _ = step()
    ok = None
    if rank == 0:  # its weak-scaling inputs are the global problem
        leaves = [rank0_dev[n].requires_grad_(True) for n in ("q", "k", "v", "g", "beta")]
        o_full, _ = ops.linear_attention("gated_deltanet", *leaves[:3], g=leaves[3], beta=leaves[4],
                                         segment_ids=rank0_dev.get("seg"))
        ok = bool(torch.equal(o_full[bs][:, :, hs], o))
    steps = 20
    blocks = [timed_block(lambda: step(), steps) for _ in range(5)]
    ms = statistics.median(blocks) / steps
    tokens = B * T
    return dict(what=f"B{B} T{T} H{H} d128 problem cut over {world} ranks by batch x heads (per rank: batch "
                     f"{loc['q'].shape[0]}, heads {loc['v'].shape[2]}), no communication",
                ms_per_step=ms, tokens_per_s=tokens / (ms * 1e-3), one_gpu_ms_per_step=one_gpu_ms_per_step,
                speedup=one_gpu_ms_per_step / ms, efficiency=one_gpu_ms_per_step / ms / world,
                shard_equals_unsharded_slice=ok)


def longctx_curve(device, rank, world, dist, timed_block, *_unused) -> dict:
    """One 1,064,960-token sequence (H16 d128, documents U[4096, 131072]) cut over the ranks along T. The one-GPU
    reference (rank 0 alone, documents as independent rows) gives the speed-up's denominator and the check: rank 0's
    shard of the sequence-parallel output against the same tokens of the one-GPU output."""
    from jax_linear_attention_b200 import ops
    from jax_linear_attention_b200.distributed import context_parallel_linear_attention, plan_pieces

    torch.cuda.empty_cache()
    dev = longctx_device_inputs(device, rank, world)
    names = ("q", "k", "v", "g", "beta")
    plan = plan_pieces(dev["seg"], 8192)

    def step():
        leaves = [dev[n].requires_grad_(True) for n in names]
        o, _ = context_parallel_linear_attention("gated_deltanet", *leaves[:3], g=leaves[3], beta=leaves[4],
                                                 segment_ids=dev["seg"], piece_len=plan)
        return o, torch.autograd.grad(o, leaves, dev["do"])

    o_cp, _ = step()
    step()
    steps = 3
    blocks = [timed_block(lambda: step(), steps) for _ in range(3)]
    ms = statistics.median(blocks) / steps
    o_cp = o_cp.detach()
    # one GPU, rank 0 only; the others wait at the next barrier
    one_ms, err, max_abs, differing, forms = None, None, None, None, None
    if rank == 0:
        one = longctx_device_inputs(device, 0, 1)

        def one_step(rows: bool):
            """The two one-GPU forms: documents as independent rows (cu_seqlens), or one packed row with segment ids,
            which the library itself cuts into pieces when that fills the SMs better."""
            leaves = [one[n].requires_grad_(True) for n in names]
            where = dict(cu_seqlens=one["cu"]) if rows else dict(segment_ids=one["seg"])
            o, _ = ops.linear_attention("gated_deltanet", *leaves[:3], g=leaves[3], beta=leaves[4], **where)
            return o, torch.autograd.grad(o, leaves, one["do"])

        o_one, _ = one_step(True)
        tl = LONG_T // world
        a, b = o_cp[:, :tl].float(), o_one.detach()[:, :tl].float()
        err = float((a - b).norm() / b.norm())
        max_abs = float((a - b).abs().max())
        differing = float((a != b).float().mean())
        del a, b, o_one
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        forms = {}
        for label, rows in (("documents_as_rows", True), ("packed_row_library_split", False)):
            one_step(rows)
            times = []
            for _ in range(3):
                torch.cuda.synchronize()
                e0.record()
                one_step(rows)
                e1.record()
                torch.cuda.synchronize()
                times.append(e0.elapsed_time(e1))
            forms[label] = statistics.median(times)
        one_ms = min(forms.values())
        del one
    torch.cuda.empty_cache()
    dist.barrier()
    return dict(what=f"one sequence of {LONG_T} tokens, H16 d128, cut over {world} ranks along T; documents in pieces of "
                     "8192 tokens joined by affine maps; NCCL send/recv of the fp32 state",
                ms_per_step=ms, tokens_per_s=LONG_T / (ms * 1e-3), one_gpu_ms_per_step=one_ms, one_gpu_forms_ms=forms,
                speedup=None if one_ms is None else one_ms / ms,
                rank0_shard_vs_one_gpu_rel_l2=err, rank0_shard_max_abs_diff=max_abs,
                rank0_shard_fraction_of_elements_differing=differing, tolerance=1e-2, within_tolerance=None if err is None else err <= 1e-2)


if __name__ == "__main__":
    main()
