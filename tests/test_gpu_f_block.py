"""GPU: a Llama-2-style decoder block on MixedQLinear layers (BASELINE config 2, reduced and full width)."""
import pytest
import torch

import torch.nn.functional as F

from oracle import kernel_path as kp
from quik_b200 import asymmetric
from quik_b200.block import QuikLlamaBlock
from quik_b200.workloads import make_layer
from tests.gpu_util import assert_device_clean, dev, rel_rms_err

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("hidden,heads,inter,seq", [(512, 8, 1408, 96), (4096, 32, 11008, 256)])
def test_block_fused_matches_unfused_and_dense(hidden, heads, inter, seq):
    blk = QuikLlamaBlock(hidden, heads, inter, fp_features=64 if hidden < 4096 else 256, seed=0, device=dev(),
                         clip=False, keep_dense=True)
    g = torch.Generator().manual_seed(1)
    x = torch.randn(1, seq, hidden, generator=g).half().to(dev())
    out = blk(x)
    assert out.shape == x.shape and torch.isfinite(out).all()
    # quantized-input caches are released after each group has been served
    assert blk.qkv_shared.qint_x is None and blk.qkv_shared.cur_group_elem == 0
    assert blk.mlp_shared.qint_x is None and blk.mlp_shared.cur_group_elem == 0
    # the reference's five-operator sequence on the same modules
    names = ["k_proj", "v_proj", "q_proj", "o_proj", "up_proj", "gate_proj", "down_proj"]
    for n in names:
        getattr(blk, n).fused = False
    unfused = blk(x)
    for n in names:
        getattr(blk, n).fused = True
    # Layer by layer the two paths agree to ~4e-6 of the RMS (tests/test_gpu_c_qlinear.py); inside a block the next
    # layer re-quantizes to 4 bits, so a value that sits on a rounding boundary can flip a code and move single
    # outputs by a fraction of a quantization step (1.1e-2 of the RMS after a 4096-wide block).  The check is
    # therefore on the RMS of the difference, with a loose cap on single elements.
    d = (out.float() - unfused.float())
    rms = unfused.float().pow(2).mean().sqrt()
    assert (d.pow(2).mean().sqrt() / rms).item() < 3e-2
    assert (d.abs().max() / rms).item() < 1.5
    # dense fp16 block with the same fake-quantized weights: differs only by the activation quantization error
    dense = blk(x, linear=lambda name, t: torch.nn.functional.linear(t, blk.dense[name]))
    # (a 4-bit code over a Gaussian row of 4096 values has a step of ~0.5 sigma, i.e. ~15% noise per layer on this
    # synthetic data; the bound only catches a wrong result, not a noisy one)
    rel = ((out.float() - dense.float()).pow(2).mean().sqrt() / dense.float().pow(2).mean().sqrt()).item()
    assert rel < 0.5, rel
    assert_device_clean()


@pytest.mark.parametrize("hidden,heads,inter,seq", [(512, 8, 1408, 96), (4096, 32, 11008, 16), (4096, 32, 11008, 256)])
def test_block_with_stacked_groups_matches_member_layers(hidden, heads, inter, seq):
    """k/v/q and up/gate as one layer each (MixedQLinear.concat): every output column is computed as in its member
    layer, so the block's output agrees with the member-wise block to the last place of a few elements at most."""
    blk = QuikLlamaBlock(hidden, heads, inter, fp_features=64 if hidden < 4096 else 256, seed=0, device=dev(), clip=False,
                         fused_producers=False)      # both sides of the comparison quantize the same torch RMSNorm output
    x = torch.randn(1, seq, hidden, generator=torch.Generator().manual_seed(2)).half().to(dev())
    separate = blk(x).clone()
    # the stacked layers alone: identical columns
    h = blk._rms_norm(x, blk.input_norm)
    blk.fuse_groups(True)
    stacked = blk._fused_groups[0](h)[0]
    members = torch.cat([blk.k_proj(h)[0], blk.v_proj(h)[0], blk.q_proj(h)[0]], dim=-1)
    d = (stacked.float() - members.float()).abs().max() / members.float().pow(2).mean().sqrt()
    assert d.item() < 2e-3
    together = blk(x)
    rms = separate.float().pow(2).mean().sqrt()
    assert ((together.float() - separate.float()).pow(2).mean().sqrt() / rms).item() < 1e-2
    assert "_fused_groups" not in "".join(blk.state_dict().keys())
    blk.fuse_groups(False)
    assert torch.equal(blk(x), separate)
    assert_device_clean()


def _buffers(m):
    buf = {"int_weight": m.int_weight.cpu(), "weights_scales": m.weights_scales.cpu(), "reduced_w": m.reduced_w.cpu(),
           "int_indices": m.int_indices.cpu(), "fp_indices": m.fp_indices.cpu(), "bias": None}
    if m.fp_features_num > 0:
        buf["fp_weight"] = m.fp_weight.cpu()
    return buf


def _oracle_block(blk, x):
    """The decoder block on the CPU: RMSNorm / RoPE / attention / SiLU in torch (the block's own arithmetic), every
    linear through the oracle's restatement of the reference kernels (quantize -> exact int GEMM -> dequantize)."""
    cpu = torch.device("cpu")
    xc = x.cpu()

    def lin(name, t):
        m = getattr(blk, name)
        return kp.mixed_linear_forward(t, _buffers(m), m.bits, round_y=False).unsqueeze(0)

    def rms(t, w):
        v = t.float()
        v = v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + blk.eps)
        return v.to(t.dtype) * w.cpu()

    b, s, _ = xc.shape
    h = rms(xc, blk.input_norm)
    k, v, q = lin("k_proj", h), lin("v_proj", h), lin("q_proj", h)
    q = q.view(b, s, blk.heads, blk.head_dim).transpose(1, 2).float()
    k = k.view(b, s, blk.kv_heads, blk.head_dim).transpose(1, 2).float()
    v = v.view(b, s, blk.kv_heads, blk.head_dim).transpose(1, 2).float()
    inv = 1.0 / (blk.rope_theta ** (torch.arange(0, blk.head_dim, 2).float() / blk.head_dim))
    ang = torch.outer(torch.arange(s).float(), inv)
    cos, sin = torch.cat([ang.cos(), ang.cos()], -1).half().float(), torch.cat([ang.sin(), ang.sin()], -1).half().float()

    def rot(t):
        hh = t.shape[-1] // 2
        return torch.cat([-t[..., hh:], t[..., :hh]], -1)
    q, k = (q * cos + rot(q) * sin).half().float(), (k * cos + rot(k) * sin).half().float()
    a = F.scaled_dot_product_attention(q, k, v, is_causal=True, scale=1.0 / blk.head_dim ** 0.5).half()
    a = a.transpose(1, 2).reshape(b, s, blk.hidden)
    xc = xc + lin("o_proj", a)
    h = rms(xc, blk.post_norm)
    up, gate = lin("up_proj", h), lin("gate_proj", h)
    act = (F.silu(gate.float()).half()) * up
    return xc + lin("down_proj", act)


@pytest.mark.parametrize("fused_producers", [True, False])
def test_block_matches_oracle_composition(fused_producers):
    """The 512-wide block against the CPU oracle's composition of the same seven linears (restatement of the
    reference kernels) with the glue in torch fp32.  A 4-bit layer re-quantizes its input, so a value on a rounding
    boundary may take the neighbouring code in one of the two computations and move single outputs by a fraction of a
    quantization step: the bound is on the RMS of the difference (and a loose cap on single elements)."""
    blk = QuikLlamaBlock(512, 8, 1408, fp_features=64, seed=0, device=dev(), clip=False, fused_producers=fused_producers)
    x = torch.randn(1, 96, 512, generator=torch.Generator().manual_seed(1)).half().to(dev())
    out = blk(x)
    for sh in (blk.qkv_shared, blk.mlp_shared, blk.o_shared, blk.down_shared):
        assert sh.qint_x is None and sh.cur_group_elem == 0
    ref = _oracle_block(blk, x)
    d = out.cpu().float() - ref.float()
    rms = ref.float().pow(2).mean().sqrt()
    assert (d.pow(2).mean().sqrt() / rms).item() < 2e-2
    assert (d.abs().max() / rms).item() < 1.0
    assert_device_clean()


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("M,K,F,bits,wide", [(300, 4096, 256, 4, True), (16, 4096, 256, 4, False), (2048, 1088, 64, 8, True),
                                            (129, 11008, 256, 8, True), (7, 608, 32, 4, False), (100, 28672, 256, 8, True)])
def test_rmsnorm_quantize_matches_norm_then_quantize(dtype, M, K, F, bits, wide):
    """RMSNorm fused into the quantizer against torch's RMSNorm followed by the plain quantizer: identical outlier
    columns up to the last place, identical codes and meta except where the two fp32 row statistics (summed in
    different orders) round a value to the neighbouring fp16 -- a few elements in a million, whole rows only when the
    row's minimum or maximum is such a value."""
    g = torch.Generator().manual_seed(M + K)
    x = torch.randn(M, K, generator=g)
    case = make_layer("t", M, K, 64, bits, F=F, seed=3, device=dev(), dtype=dtype, clip=False)
    x[:, case.fp_indices] *= 20
    x = (x * 1.7).to(dtype).to(dev())
    w = (1.0 + 0.1 * torch.randn(K, generator=g)).to(dtype).to(dev())
    eps = 1e-5
    i16, f16 = case.module._idx16()
    v = x.float()
    normed = (v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + eps)).to(dtype) * w
    q0, m0, f0 = asymmetric.quantize_u16(normed.contiguous(), i16, f16, bits, wide)
    q1, m1, f1 = asymmetric.rmsnorm_quantize_u16(x, w, eps, i16, f16, bits, wide)
    torch.cuda.synchronize()
    assert q1.shape == q0.shape and m1.shape == m0.shape and f1.shape == f0.shape
    ulp = 2.0 ** (-10 if dtype == torch.float16 else -7)
    assert ((f1.float() - f0.float()).abs() <= 1.01 * ulp * f0.float().abs() + 1e-6).all()
    assert (f1 != f0).float().mean().item() < 5e-3
    rows_same = (m1.view(M, 2) == m0.view(M, 2)).all(dim=1)
    assert rows_same.float().mean().item() > 0.97
    if rows_same.any():
        same = (q1[rows_same] == q0[rows_same]).float().mean().item()
        assert same > 1 - 1e-3, same
    # rows whose meta moved by a unit in the last place are still self-consistent: dequantized values agree
    assert ((m1.float() - m0.float()).abs() <= 2 * ulp * m0.float().abs() + 1e-6).all()
    assert_device_clean()


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("M,K,F,bits,wide", [(300, 11008, 256, 8, True), (16, 1408, 64, 8, True), (2048, 1408, 64, 4, True),
                                            (9, 608, 32, 4, False)])
def test_silu_mul_quantize_matches_activation_then_quantize(dtype, M, K, F, bits, wide):
    """SiLU(gate) * up fused into the quantizer against torch's F.silu(gate) * up followed by the plain quantizer
    (elementwise producers: no reduction order is involved, the exponential's last place is the only difference)."""
    g = torch.Generator().manual_seed(M + K + 1)
    gate = (2.0 * torch.randn(M, K, generator=g)).to(dtype).to(dev())
    up = torch.randn(M, K, generator=g).to(dtype).to(dev())
    case = make_layer("t", M, K, 64, bits, F=F, seed=4, device=dev(), dtype=dtype, clip=False)
    i16, f16 = case.module._idx16()
    act = (torch.nn.functional.silu(gate) * up).contiguous()
    q0, m0, f0 = asymmetric.quantize_u16(act, i16, f16, bits, wide)
    q1, m1, f1 = asymmetric.silu_mul_quantize_u16(gate, up, i16, f16, bits, wide)
    torch.cuda.synchronize()
    ulp = 2.0 ** (-10 if dtype == torch.float16 else -7)
    assert ((f1.float() - f0.float()).abs() <= 2.01 * ulp * f0.float().abs() + 1e-6).all()
    rows_same = (m1.view(M, 2) == m0.view(M, 2)).all(dim=1)
    assert rows_same.float().mean().item() > 0.97
    if rows_same.any():
        assert (q1[rows_same] == q0[rows_same]).float().mean().item() > 1 - 1e-3
    assert_device_clean()


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("heads,kv_heads,head_dim,seq", [(8, 8, 64, 33), (32, 8, 128, 257), (4, 2, 16, 5)])
def test_rotary_inplace_is_bit_identical_to_the_torch_expression(dtype, heads, kv_heads, head_dim, seq):
    """quik_rotary_inplace against x * cos + rotate_half(x) * sin in torch (transformers' apply_rotary_pos_emb
    arithmetic): every product and sum rounds to the storage type in both, so the bits agree."""
    blk = QuikLlamaBlock.__new__(QuikLlamaBlock)
    torch.nn.Module.__init__(blk)
    blk.heads, blk.kv_heads, blk.head_dim, blk.rope_theta, blk._rope_cache = heads, kv_heads, head_dim, 10000.0, {}
    g = torch.Generator().manual_seed(5)
    q = torch.randn(seq, heads * head_dim, generator=g).to(dtype).cuda()
    k = torch.randn(seq, kv_heads * head_dim, generator=g).to(dtype).cuda()
    qv = q.view(1, seq, heads, head_dim).transpose(1, 2)
    kv = k.view(1, seq, kv_heads, head_dim).transpose(1, 2)
    rq, rk = blk._rope(qv, kv)
    want_q = rq.transpose(1, 2).reshape(seq, -1).clone()
    want_k = rk.transpose(1, 2).reshape(seq, -1).clone()
    blk._rope_inplace(q, k, seq)
    torch.cuda.synchronize()
    assert torch.equal(q, want_q)
    assert torch.equal(k, want_k)


def test_block_with_and_without_fused_rotary_agree_bitwise():
    blk = QuikLlamaBlock(512, 8, 1024, seed=3)
    x = torch.randn(1, 96, 512, generator=torch.Generator().manual_seed(1)).half().cuda()
    a = blk(x).clone()
    blk.fused_rope = False
    b = blk(x)
    torch.cuda.synchronize()
    assert torch.equal(a, b)
