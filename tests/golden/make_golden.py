"""Regenerates the golden fixtures in this directory FROM THE REFERENCE PROJECT.

Run in a container where the reference checkout is available:

    python tests/golden/make_golden.py /path/to/reference

It imports the reference's own `kernelforge.quantize` (pure torch, CPU) and the FP32
oracles of its test-suite (`reference_general`, tests/test_attention.py:217-226;
`x.float() @ dequantize(qw, fp32).T`, tests/test_gemm.py:32) and stores their outputs for
small seeded inputs as .npz files.  The fixtures travel with the repository; the
reference does not, so nothing else may import it.
"""

from __future__ import annotations

import importlib.util
import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent


def _ref_modules(ref_root: Path):
    sys.path.insert(0, str(ref_root))
    from kernelforge import quantize as kq  # noqa: E402  (reference package)
    spec = importlib.util.spec_from_file_location("ref_test_attention", ref_root / "tests" / "test_attention.py")
    ta = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(ta)
    return kq, ta


def quant_cases(kq):
    g = torch.Generator().manual_seed(1234)
    for group in (64, 128):
        w = torch.randn(24, 512, generator=g) * 0.02
        w[3, :group] = 0.0                       # all-zero group -> scale 1
        w[4, :group] = 0.0
        w[4, 5] = -3.5                           # absmax maps to -7
        w[4, 9] = 1.0
        # exact half steps with scale exactly 1 (absmax 7): rint must round half to even
        w[5, :group] = 0.0
        ties = torch.tensor([7.0, 0.5, 1.5, 2.5, -0.5, -1.5, -2.5, 6.5, -6.5, 3.5, -3.5, 4.5])
        w[5, : ties.numel()] = ties
        w[6, :group] = torch.randn(group, generator=g) * 1e-7   # below fp16-normal clamp
        w[7, group:2 * group] = torch.randn(group, generator=g) * 30.0
        for tag, wt in (("f32", w), ("f16", w.half()), ("bf16", w.bfloat16())):
            qw = kq.quantize_weight(wt, group)
            q, s = kq.quantize_int4(wt, group)
            assert torch.equal(kq.unpack_int4(qw.packed), q)
            np.savez_compressed(
                HERE / f"quant_g{group}_{tag}.npz",
                w=wt.float().numpy(), q=q.numpy(), packed=qw.packed.numpy(), scales=qw.scales.numpy(),
                deq32=kq.dequantize(qw, torch.float32).numpy(), deq16=kq.dequantize(qw, torch.float16).numpy(),
                group=np.int32(group))


def linear_cases(kq):
    g = torch.Generator().manual_seed(99)
    for m, n, k, group in ((1, 64, 256, 128), (3, 129, 256, 128), (8, 72, 512, 64), (17, 128, 1024, 128)):
        w = torch.randn(n, k, generator=g) * 0.02
        x = torch.randn(m, k, generator=g).half()
        qw = kq.quantize_weight(w, group)
        ref = x.float() @ kq.dequantize(qw, torch.float32).T
        np.savez_compressed(HERE / f"int4_linear_m{m}_n{n}_k{k}_g{group}.npz", x=x.numpy(), packed=qw.packed.numpy(),
                            scales=qw.scales.numpy(), ref=ref.numpy(), group=np.int32(group))


def attention_cases(ta):
    for (h, hk, nq, nk, d, causal) in ((4, 4, 16, 16, 64, False), (4, 2, 1, 37, 64, True), (8, 2, 7, 64, 128, True),
                                       (4, 1, 65, 130, 64, True), (2, 2, 130, 131, 128, False),
                                       (8, 1, 1, 300, 64, False)):
        g = torch.Generator().manual_seed(nq * 31 + nk + h + d)
        q = torch.randn(2, h, nq, d, generator=g).half()
        k = torch.randn(2, hk, nk, d, generator=g).half()
        v = torch.randn(2, hk, nk, d, generator=g).half()
        ref = ta.reference_general(q, k, v, causal)
        np.savez_compressed(HERE / f"attn_h{h}_hk{hk}_nq{nq}_nk{nk}_d{d}_{'causal' if causal else 'full'}.npz",
                            q=q.numpy(), k=k.numpy(), v=v.numpy(), ref=ref.numpy(), causal=np.bool_(causal))
    # the square-mask oracle with an explicit scale (tests/test_attention.py:33-41)
    g = torch.Generator().manual_seed(3)
    q, k, v = (torch.randn(1, 2, 50, 64, generator=g).half() for _ in range(3))
    ref = ta.reference_attention(q, k, v, True, 0.05)
    np.savez_compressed(HERE / "attn_square_scale0.05_causal.npz", q=q.numpy(), k=k.numpy(), v=v.numpy(),
                        ref=ref.numpy(), causal=np.bool_(True), scale=np.float32(0.05))


def main():
    if len(sys.argv) != 2:
        sys.exit("usage: python tests/golden/make_golden.py <path of a checkout of the reference repository>")
    ref_root = Path(sys.argv[1])
    kq, ta = _ref_modules(ref_root)
    torch.set_num_threads(4)
    quant_cases(kq)
    linear_cases(kq)
    attention_cases(ta)
    print("wrote", len(list(HERE.glob('*.npz'))), "fixtures to", HERE)


if __name__ == "__main__":
    main()
