"""Generate the golden fixtures in this folder from the reference's own Python.

Run once, where the reference checkout is available:

    python tests/golden/make_golden.py /path/to/QUIK

It imports, unmodified, ``experiments/qlinear.py`` (``pack_to_i4``, ``two_compl``,
``MixedQLinear.from_float``) and ``experiments/quant_sim.py`` (``WeightQuantizer``,
``ActQuantWrapper``) and records their outputs on small seeded inputs.  The
reference's CUDA operators cannot run without its compiled extension and a GPU,
so ``qlinear.py`` is imported with an empty stand-in for the ``quik`` module and
with ``Tensor.cuda()`` made a no-op; only code that is pure torch is executed.
The fixtures are a few KB each and are read by ``tests/test_oracle_golden.py``.
"""
import os
import sys
import types

import torch


def main(ref_root: str) -> None:
    here = os.path.dirname(os.path.abspath(__file__))
    sys.path.insert(0, os.path.join(ref_root, "experiments"))
    sys.modules.setdefault("quik", types.ModuleType("quik"))      # CUDA ops are never called below
    torch.Tensor.cuda = lambda self, *a, **k: self                # from_float calls .cuda()
    import qlinear as ref_qlinear                                 # noqa: E402
    import quant_sim as ref_sim                                   # noqa: E402

    out = {}

    # ---- pack_to_i4 / two_compl (qlinear.py:11-18)
    g = torch.Generator().manual_seed(11)
    vals = torch.randint(-8, 8, (6, 32), generator=g, dtype=torch.int8)
    out["pack"] = {"vals": vals, "packed": ref_qlinear.pack_to_i4(vals),
                   "two_compl": ref_qlinear.two_compl(vals, 4)}

    # ---- MixedQLinear.from_float buffers (qlinear.py:150-199)
    cases = []
    for bits in (4, 8):
        for dtype in (torch.float16, torch.bfloat16):
            for with_bias in (False, True):
                for nfp in (0, 6):
                    g = torch.Generator().manual_seed(100 + bits + nfp)
                    n, k = 12, 40
                    lin = torch.nn.Linear(k, n, bias=with_bias)
                    w = (0.02 * torch.randn(n, k, generator=g)).to(dtype)
                    if with_bias:
                        lin.bias.data = torch.randn(n, generator=g)
                    maxq = 7 if bits == 4 else 127
                    scales = (w.float().abs().max(dim=1, keepdim=True)[0] / maxq)
                    fp_idx = torch.randperm(k, generator=g)[:nfp] if nfp else None
                    mod = ref_qlinear.MixedQLinear.from_float(lin, w, scales, fp_indices=fp_idx, bits=bits)
                    bufs = {name: b.clone() for name, b in mod.named_buffers()}
                    cases.append({"bits": bits, "dtype": dtype, "weight": w, "scales": scales,
                                  "fp_indices": fp_idx, "bias": lin.bias.data.clone() if with_bias else None,
                                  "buffers": bufs, "bias_is_none": mod.bias is None})
    out["from_float"] = cases

    # ---- weight RTN + clipping (quant_sim.py:30-136) and the fake-quant layer (quant_sim.py:193-257)
    fq = []
    for bits in (4, 8):
        for nfp in (0, 8):
            g = torch.Generator().manual_seed(7 + bits + nfp)
            n, k, m = 16, 64, 9
            w = 0.02 * torch.randn(n, k, generator=g)
            x = torch.randn(m, k, generator=g)
            scales_in = torch.zeros(k)
            if nfp:
                cols = torch.randperm(k, generator=g)[:nfp]
                x[:, cols] *= 20
                scales_in[cols] = 1.0
            x = x.half()
            wq = ref_sim.WeightQuantizer()
            wq.configure(bits, perchannel=True, sym=True, mse=True)
            lin = torch.nn.Linear(k, n, bias=False)
            wrap = ref_sim.ActQuantWrapper(lin)
            wrap.fp_features_configure(scales_in, nfp)
            wrap.quantizer.configure(bits)
            int_cols = wrap.quantized_feature_idx
            wq.find_params(w[:, int_cols])
            w_dq = w.clone()
            w_dq[:, int_cols] = wq.quantize(w[:, int_cols])
            lin.weight.data = w_dq.half()
            lin.half()
            with torch.no_grad():
                y = wrap(x)
            fq.append({"bits": bits, "nfp": nfp, "w": w, "x": x, "act_scales": scales_in,
                       "w_scale": wq.scale.clone(), "w_dq": w_dq, "y": y})
    out["fakequant"] = fq

    torch.save(out, os.path.join(here, "reference_python.pt"))
    print("wrote", os.path.join(here, "reference_python.pt"))


if __name__ == "__main__":
    ref_dir = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("QUIK_REFERENCE_DIR")
    if not ref_dir:
        raise SystemExit("usage: python tests/golden/make_golden.py <path of the reference checkout> "
                         "(or set QUIK_REFERENCE_DIR)")
    main(ref_dir)
