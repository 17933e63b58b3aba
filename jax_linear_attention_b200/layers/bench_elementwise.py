"""Device times of the element-wise layer kernels around the op, forward and backward, at the shapes of the benchmark
workloads: ``python -m jax_linear_attention_b200.layers.bench_elementwise [--only gates|conv|norm] [--steps N]``.

Each case builds its tensors on the device, calls the layer function and its backward ``--warmup`` times and then
``--steps`` times between CUDA events, writing a buffer larger than L2 before every call so that the inputs come from
HBM. The host cost of a call (a ``torch.autograd.Function`` and a ctypes call, 30-60 us) is inside these times; the
kernels' own durations come from running the same command under a one-pass launch list
(``ncu --metrics gpu__time_duration.sum --clock-control none -k regex:<kernel> ...``)."""

from __future__ import annotations

import argparse

import torch

from . import gate_prologue, gated_rms_norm, short_conv


def _timed(fwd, bwd, steps, warmup, flush):
    for _ in range(warmup):
        bwd(fwd())
    torch.cuda.synchronize()
    tf = tb = 0.0
    for _ in range(steps):
        flush.zero_()
        e = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
        e[0].record()
        out = fwd()
        e[1].record()
        bwd(out)
        e[2].record()
        torch.cuda.synchronize()
        tf += e[0].elapsed_time(e[1])
        tb += e[1].elapsed_time(e[2])
    return tf / steps, tb / steps


def cases(dev):
    bf16 = torch.bfloat16
    # gate activations: Gated DeltaNet (one decay per head) and KDA (one per key channel)
    for shape, name in (((8, 2048, 16), "gates GDN B8 T2048 H16"), ((4, 4096, 16, 128), "gates KDA B4 T4096 H16 K128")):
        a = torch.randn(shape, device=dev, dtype=bf16, requires_grad=True)
        b = torch.randn(shape[:3], device=dev, dtype=bf16, requires_grad=True)
        a_log = torch.zeros(16, device=dev, requires_grad=True)
        dt_bias = torch.zeros(shape[2:], device=dev, requires_grad=True)
        dg, dbeta = torch.randn(shape, device=dev), torch.randn(shape[:3], device=dev)
        nbytes = (a.numel() + b.numel()) * (2 + 4), (a.numel() + b.numel()) * (2 + 4 + 2)
        yield ("gates", name, lambda a=a, b=b, a_log=a_log, dt_bias=dt_bias: gate_prologue(a, a_log, dt_bias, b),
               lambda out, a=a, b=b, a_log=a_log, dt_bias=dt_bias, dg=dg, dbeta=dbeta:
               torch.autograd.grad(list(out), [a, a_log, dt_bias, b], [dg, dbeta]), nbytes)
    # q (or k) prologue of a Gated DeltaNet layer: short conv, SiLU, L2 norm per head, packed documents
    B, T, C, K = 8, 2048, 2048, 4
    x = torch.randn(B, T, C, device=dev, dtype=bf16, requires_grad=True)
    w = (torch.randn(C, K, device=dev) * 0.5).requires_grad_(True)
    seg = (torch.arange(T, device=dev)[None] // 700).expand(B, T).to(torch.int32).contiguous()
    dy = torch.randn(B, T, C, device=dev, dtype=bf16)
    yield ("conv", "short conv + SiLU + L2 norm B8 T2048 C2048 K4 head 128",
           lambda: short_conv(x, w, head_dim=128, segment_ids=seg)[0],
           lambda y: torch.autograd.grad([y], [x, w], [dy]), (x.numel() * 4, x.numel() * 6))
    # output norm of a Gated DeltaNet layer (one group per head) and of a Mamba-2 layer (one group per token)
    for shape, group, nbg, name in (((8, 2048, 16, 128), None, True, "gated RMS norm B8 T2048 H16 V128"),
                                    ((8, 2048, 4096), 4096, False, "gated RMS norm B8 T2048 d_inner 4096")):
        o = torch.randn(shape, device=dev, dtype=bf16, requires_grad=True)
        z = torch.randn(shape, device=dev, dtype=bf16, requires_grad=True)
        wn = torch.ones(shape[-1], device=dev, requires_grad=True)
        dyn = torch.randn(shape, device=dev, dtype=bf16)
        yield ("norm", name,
               lambda o=o, z=z, wn=wn, nbg=nbg, group=group: gated_rms_norm(o, z, wn, norm_before_gate=nbg, group_size=group),
               lambda y, o=o, z=z, wn=wn, dyn=dyn: torch.autograd.grad([y], [o, z, wn], [dyn]),
               (o.numel() * 6, o.numel() * 10))


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__.splitlines()[0])
    ap.add_argument("--only", choices=("gates", "conv", "norm"), default=None)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    args = ap.parse_args()
    if not torch.cuda.is_available():
        raise SystemExit("needs a CUDA device: the layer kernels have no CPU fallback")
    dev = torch.device("cuda")
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    for kind, name, fwd, bwd, (fb, bb) in cases(dev):
        if args.only and kind != args.only:
            continue
        tf, tb = _timed(fwd, bwd, args.steps, args.warmup, flush)
        print(f"{name}: fwd {tf * 1e3:.0f} us ({fb / tf / 1e6:.0f} GB/s), bwd {tb * 1e3:.0f} us ({bb / tb / 1e6:.0f} GB/s)"
              " incl. the host side of the call")


if __name__ == "__main__":
    main()
