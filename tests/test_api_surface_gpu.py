"""The parts of the Python surface that the kernels' parity tests do not reach: the fake (meta) registrations of the
custom ops, which torch.compile traces instead of running the kernels (reference:
flash_attn_npu/flash_attn_npu_interface.py:104-131, :188-224, :281-315 with the 128-rounded softmax_d, :385-426), and
the two packed variants of the packed-sequence API (flash_attn_varlen_qkvpacked_func :1186,
flash_attn_varlen_kvpacked_func :1252), forward and backward."""
import pytest
import torch

from oracle import attention_oracle as orc
from parity import assert_lse, assert_within

pytestmark = pytest.mark.gpu
CHECKS = ("test_schema", "test_faketensor")


def _dense(b=2, sq=200, sk=264, h=4, hkv=2, d=64, dt=torch.bfloat16):
    q, do = torch.randn(b, sq, h, d, device="cuda").to(dt), torch.randn(b, sq, h, d, device="cuda").to(dt)
    k, v = torch.randn(b, sk, hkv, d, device="cuda").to(dt), torch.randn(b, sk, hkv, d, device="cuda").to(dt)
    return q, k, v, do


def _packed(lens_q=(70, 1, 200), lens_k=(70, 40, 333), h=4, hkv=2, d=64, dt=torch.bfloat16):
    cu_q = torch.tensor([0] + torch.tensor(lens_q).cumsum(0).tolist(), dtype=torch.int32, device="cuda")
    cu_k = torch.tensor([0] + torch.tensor(lens_k).cumsum(0).tolist(), dtype=torch.int32, device="cuda")
    q, do = torch.randn(sum(lens_q), h, d, device="cuda").to(dt), torch.randn(sum(lens_q), h, d, device="cuda").to(dt)
    k, v = torch.randn(sum(lens_k), hkv, d, device="cuda").to(dt), torch.randn(sum(lens_k), hkv, d, device="cuda").to(dt)
    return q, k, v, do, cu_q, cu_k, max(lens_q), max(lens_k)


def test_fake_registrations_of_the_v2_ops_match_the_kernels():
    import flash_attn_npu  # noqa: F401  (registers the ops)
    ops = torch.ops.flash_attn_npu
    q, k, v, do = _dense()
    scale = q.shape[-1] ** -0.5
    torch.library.opcheck(ops._flash_attn_forward, (q, k, v, 0.0, scale, True, -1, -1, 0.0, None, False), test_utils=CHECKS)
    out, lse, _, rng = ops._flash_attn_forward(q, k, v, 0.0, scale, True, -1, -1, 0.0, None, False)
    dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
    torch.library.opcheck(ops._flash_attn_backward, (do, q, k, v, out, lse, dq, dk, dv, 0.0, scale, True, -1, -1, 0.0, None, False),
                          test_utils=CHECKS)
    d_ = ops._flash_attn_backward(do, q, k, v, out, lse, dq, dk, dv, 0.0, scale, True, -1, -1, 0.0, None, False)
    assert d_.shape == (q.shape[0], q.shape[2], 256) and d_.dtype == torch.float32     # seqlen 200 rounded up to 128s
    qp, kp, vp, dop, cu_q, cu_k, mq, mk = _packed()
    torch.library.opcheck(ops._flash_attn_varlen_forward, (qp, kp, vp, cu_q, cu_k, mq, mk, 0.0, scale, True), test_utils=CHECKS)
    outp, lsep, _, _ = ops._flash_attn_varlen_forward(qp, kp, vp, cu_q, cu_k, mq, mk, 0.0, scale, True)
    assert lsep.shape == (qp.shape[1], qp.shape[0])
    dqp, dkp, dvp = torch.empty_like(qp), torch.empty_like(kp), torch.empty_like(vp)
    args = (dop, qp, kp, vp, outp, lsep, dqp, dkp, dvp, cu_q, cu_k, mq, mk, 0.0, scale, True, -1, -1, 0.0, None, False)
    torch.library.opcheck(ops._flash_attn_varlen_backward, args, test_utils=CHECKS)
    d_ = ops._flash_attn_varlen_backward(*args)
    assert d_.shape == (qp.shape[1], qp.shape[0] + 128 * 3)


def test_fake_registrations_of_the_v3_ops_match_the_kernels():
    import flash_attn_npu_3  # noqa: F401
    ops = torch.ops.flash_attn_npu_3
    q, k, v, do = _dense()
    scale = q.shape[-1] ** -0.5
    kw = dict(softmax_scale=scale, causal=True)
    torch.library.opcheck(ops._flash_attn_forward, (q, k, v), kw, test_utils=CHECKS)
    out, lse, _, _ = ops._flash_attn_forward(q, k, v, **kw)
    dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
    kwb = dict(dq=dq, dk=dk, dv=dv, softmax_scale=scale, is_causal=True)
    torch.library.opcheck(ops._flash_attn_backward, (do, q, k, v, out, lse), kwb, test_utils=CHECKS)
    qp, kp, vp, dop, cu_q, cu_k, mq, mk = _packed()
    kwp = dict(cu_seqlens_q=cu_q, cu_seqlens_k=cu_k, max_seqlen_q=mq, max_seqlen_k=mk, softmax_scale=scale, causal=True)
    torch.library.opcheck(ops._flash_attn_forward, (qp, kp, vp), kwp, test_utils=CHECKS)


def test_traced_with_fake_tensors_gives_the_eager_shapes():
    """What torch.compile sees: the whole public function run on FakeTensors, no kernel launched."""
    import flash_attn_npu as fa
    from torch._subclasses.fake_tensor import FakeTensorMode
    q, k, v, _ = _dense()
    real = fa.flash_attn_func(q, k, v, causal=True, return_attn_probs=True)
    with FakeTensorMode(allow_non_fake_inputs=False) as mode:
        fq, fk, fv = (mode.from_tensor(t) for t in (q, k, v))
        fake = fa.flash_attn_func(fq, fk, fv, causal=True, return_attn_probs=True)
    assert fake[0].shape == real[0].shape and fake[0].dtype == real[0].dtype
    assert fake[1].shape == real[1].shape and fake[1].dtype == torch.float32


@pytest.mark.parametrize("causal", [False, True])
def test_varlen_qkvpacked_forward_and_backward(causal):
    import flash_attn_npu as fa
    lens = [130, 1, 257, 64]
    cu = torch.tensor([0] + torch.tensor(lens).cumsum(0).tolist(), dtype=torch.int32)
    h, d = 3, 128
    qkv = (torch.rand(sum(lens), 3, h, d) * 2 - 1).bfloat16()
    do = (torch.rand(sum(lens), h, d) * 2 - 1).bfloat16()
    q, k, v = qkv[:, 0], qkv[:, 1], qkv[:, 2]
    scale = d ** -0.5
    lp_o, _ = orc.attention_varlen_fwd(q, k, v, cu, cu, scale, causal)
    f_o, f_l = orc.attention_varlen_fwd(q.float(), k.float(), v.float(), cu, cu, scale, causal, data_type=torch.float32)
    lp = orc.attention_varlen_bwd(q, k, v, do, f_l, cu, cu, scale, causal)
    f32 = orc.attention_varlen_bwd(q.float(), k.float(), v.float(), do.float(), f_l, cu, cu, scale, causal)
    x = qkv.cuda().requires_grad_(True)
    out, lse, _ = fa.flash_attn_varlen_qkvpacked_func(x, cu.cuda(), max(lens), causal=causal, return_attn_probs=True)
    (g,) = torch.autograd.grad(out, (x,), do.cuda())
    assert_within("out", out.detach().cpu(), lp_o, f_o)
    assert_lse(lse, f_l)
    for i, name in enumerate(("dq", "dk", "dv")):
        assert_within(name, g[:, i].cpu(), lp[i], f32[i], roundings=3)


@pytest.mark.parametrize("causal", [False, True])
def test_varlen_kvpacked_forward_and_backward(causal):
    import flash_attn_npu as fa
    lens_q, lens_k = [100, 2, 129], [180, 77, 129]
    cu_q = torch.tensor([0] + torch.tensor(lens_q).cumsum(0).tolist(), dtype=torch.int32)
    cu_k = torch.tensor([0] + torch.tensor(lens_k).cumsum(0).tolist(), dtype=torch.int32)
    h, hkv, d = 6, 2, 64
    q = (torch.rand(sum(lens_q), h, d) * 2 - 1).to(torch.float16)
    kv = (torch.rand(sum(lens_k), 2, hkv, d) * 2 - 1).to(torch.float16)
    do = (torch.rand(sum(lens_q), h, d) * 2 - 1).to(torch.float16)
    k, v = kv[:, 0], kv[:, 1]
    scale = d ** -0.5
    lp_o, _ = orc.attention_varlen_fwd(q, k, v, cu_q, cu_k, scale, causal)
    f_o, f_l = orc.attention_varlen_fwd(q.float(), k.float(), v.float(), cu_q, cu_k, scale, causal, data_type=torch.float32)
    lp = orc.attention_varlen_bwd(q, k, v, do, f_l, cu_q, cu_k, scale, causal)
    f32 = orc.attention_varlen_bwd(q.float(), k.float(), v.float(), do.float(), f_l, cu_q, cu_k, scale, causal)
    qc, kvc = q.cuda().requires_grad_(True), kv.cuda().requires_grad_(True)
    out, lse, _ = fa.flash_attn_varlen_kvpacked_func(qc, kvc, cu_q.cuda(), cu_k.cuda(), max(lens_q), max(lens_k), causal=causal,
                                                     return_attn_probs=True)
    gq, gkv = torch.autograd.grad(out, (qc, kvc), do.cuda())
    assert_within("out", out.detach().cpu(), lp_o, f_o)
    assert_lse(lse, f_l)
    assert_within("dq", gq.cpu(), lp[0], f32[0], roundings=3)
    assert_within("dk", gkv[:, 0].cpu(), lp[1], f32[1], roundings=3)
    assert_within("dv", gkv[:, 1].cpu(), lp[2], f32[2], roundings=3)
