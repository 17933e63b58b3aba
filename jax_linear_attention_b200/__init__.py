"""B200 (sm_100a) kernels for the chunkwise gated delta rule family behind the ``jla.ops`` call surface.

    from jax_linear_attention_b200 import ops
    o, final_state = ops.linear_attention("gated_deltanet", q, k, v, g=g, beta=beta)

The compute lives in ``libjla_b200.so`` (hand-written CUDA, C ABI in ``include/jla_b200.h``); this package
is the host side: the dispatcher and per-kind functions of ``jla.ops``, the Mamba-2 SSD mapping, batch x heads
sharding and the sequence-parallel mode. Tensors are torch CUDA tensors (device memory and streams only).
"""

__version__ = "0.1.0"
