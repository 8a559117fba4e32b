"""tcgen05 attention vs fp32 PyTorch: causal / non-causal, GQA, ragged lengths, GRPO prefix sharing."""

import math

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _rand(shape, seed, scale=1.0):
    g = torch.Generator(device=DEV).manual_seed(seed)
    return (torch.randn(shape, device=DEV, generator=g) * scale).to(torch.bfloat16)


@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("b,s,hq,hkv", [(2, 128, 4, 4), (1, 384, 8, 2), (3, 200, 4, 1), (2, 77, 2, 2)])
def test_attn_op_matches_sdpa(causal, b, s, hq, hkv):
    from rl_engine.kernels.ops.pytorch.attention import NativeAttentionOp
    from rl_engine.kernels.ops.sm100.attention import FlashAttentionSM100Op

    q, k, v = _rand((b, s, hq, 128), 1), _rand((b, s, hkv, 128), 2), _rand((b, s, hkv, 128), 3)
    got = FlashAttentionSM100Op()(q, k, v, causal=causal)
    want = NativeAttentionOp()(q.float(), k.float(), v.float(), causal=causal)
    assert (got.float() - want).abs().max().item() < 2e-2
    assert torch.equal(got, FlashAttentionSM100Op()(q, k, v, causal=causal))


@pytest.mark.parametrize("bs,G,lq,lkv", [(1, 4, 128, 256), (2, 3, 192, 1000), (1, 8, 64, 130)])
def test_prefix_shared_noncausal(bs, G, lq, lkv):
    from rl_engine.kernels.ops.pytorch.attention import NativePrefixSharedAttentionOp
    from rl_engine.kernels.ops.sm100.attention import PrefixSharedAttentionSM100Op

    q, k, v = _rand((bs, G, lq, 128), 4), _rand((bs, lkv, 128), 5), _rand((bs, lkv, 128), 6)
    got = PrefixSharedAttentionSM100Op()(q, k, v)
    want = NativePrefixSharedAttentionOp()(q.float(), k.float(), v.float())
    assert (got.float() - want).abs().max().item() < 2e-2


@pytest.mark.parametrize("P,G,L,hq,hkv", [(256, 4, 128, 4, 2), (100, 3, 70, 8, 2), (1024, 2, 512, 4, 1)])
def test_grpo_group_attention_forward_and_backward(P, G, L, hq, hkv):
    from rl_engine.kernels.ops.pytorch.attention import grouped_prefix_causal_attention_reference
    from rl_engine.kernels.ops.sm100.attention import grouped_prefix_attention, grpo_group_layout, packed_attention_forward

    T = P + G * L
    q, k, v = _rand((T, hq, 128), 7), _rand((T, hkv, 128), 8), _rand((T, hkv, 128), 9)
    layout = grpo_group_layout(P, G, L, DEV)
    out, lse = packed_attention_forward(q, k, v, layout)
    # completions: oracle with explicit prefix + causal suffix
    want, want_lse = grouped_prefix_causal_attention_reference(
        q[P:].reshape(G, L, hq, 128), k[:P], v[:P], k[P:].reshape(G, L, hkv, 128), v[P:].reshape(G, L, hkv, 128)
    )
    assert (out[P:].reshape(G, L, hq, 128).float() - want).abs().max().item() < 2e-2
    got_lse = lse[:, P:].reshape(hq, G, L).permute(1, 0, 2)
    assert (got_lse - want_lse).abs().max().item() < 2e-2
    # prompt rows: plain causal attention
    qp = q[:P].float().transpose(0, 1)
    kp = k[:P].float().transpose(0, 1).repeat_interleave(hq // hkv, 0)
    vp = v[:P].float().transpose(0, 1).repeat_interleave(hq // hkv, 0)
    ref_p = torch.nn.functional.scaled_dot_product_attention(qp, kp, vp, is_causal=True).transpose(0, 1)
    assert (out[:P].float() - ref_p).abs().max().item() < 2e-2

    # gradients vs autograd through the fp32 oracle
    qa, ka, va = (t.clone().requires_grad_(True) for t in (q, k, v))
    dout = _rand((T, hq, 128), 10)
    grouped_prefix_attention(qa, ka, va, P, G, L).backward(dout)
    qb, kb, vb = (t.clone().float().requires_grad_(True) for t in (q, k, v))
    oc, _ = grouped_prefix_causal_attention_reference(
        qb[P:].reshape(G, L, hq, 128), kb[:P], vb[:P], kb[P:].reshape(G, L, hkv, 128), vb[P:].reshape(G, L, hkv, 128)
    )
    op = torch.nn.functional.scaled_dot_product_attention(
        qb[:P].transpose(0, 1), kb[:P].transpose(0, 1).repeat_interleave(hq // hkv, 0),
        vb[:P].transpose(0, 1).repeat_interleave(hq // hkv, 0), is_causal=True,
    ).transpose(0, 1)
    torch.cat([op, oc.reshape(G * L, hq, 128)]).backward(dout.float())
    for got, want in ((qa.grad, qb.grad), (ka.grad, kb.grad), (va.grad, vb.grad)):
        scale = want.abs().max().item()
        assert (got.float() - want).abs().max().item() / scale < 3e-2


@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("b,s,hq,hkv", [(2, 128, 4, 4), (1, 320, 8, 2), (2, 77, 4, 1)])
def test_attn_op_backward_matches_sdpa(causal, b, s, hq, hkv):
    from rl_engine.kernels.ops.pytorch.attention import NativeAttentionOp
    from rl_engine.kernels.ops.sm100.attention import FlashAttentionSM100Op

    q, k, v = _rand((b, s, hq, 128), 11), _rand((b, s, hkv, 128), 12), _rand((b, s, hkv, 128), 13)
    dout = _rand((b, s, hq, 128), 14)
    qa, ka, va = (t.clone().requires_grad_(True) for t in (q, k, v))
    FlashAttentionSM100Op()(qa, ka, va, causal=causal).backward(dout)
    qb, kb, vb = (t.clone().float().requires_grad_(True) for t in (q, k, v))
    NativeAttentionOp()(qb, kb, vb, causal=causal).backward(dout.float())
    for got, want in ((qa.grad, qb.grad), (ka.grad, kb.grad), (va.grad, vb.grad)):
        scale = want.abs().max().item()
        assert (got.float() - want).abs().max().item() / scale < 3e-2
    # bitwise reproducible
    q2, k2, v2 = (t.clone().requires_grad_(True) for t in (q, k, v))
    FlashAttentionSM100Op()(q2, k2, v2, causal=causal).backward(dout)
    assert torch.equal(qa.grad, q2.grad) and torch.equal(ka.grad, k2.grad) and torch.equal(va.grad, v2.grad)


def test_split_key_tiles_reduce_in_order():
    """A prompt shared by many completions forces split dK/dV items plus the ordered reduction."""
    from rl_engine.kernels.ops.pytorch.attention import grouped_prefix_causal_attention_reference
    from rl_engine.kernels.ops.sm100.attention import grouped_prefix_attention

    P, G, L, hq, hkv = 128, 40, 128, 2, 1   # 80 query blocks per prefix tile > 64 per item
    T = P + G * L
    q, k, v = _rand((T, hq, 128), 21), _rand((T, hkv, 128), 22), _rand((T, hkv, 128), 23)
    dout = _rand((T, hq, 128), 24)
    qa, ka, va = (t.clone().requires_grad_(True) for t in (q, k, v))
    grouped_prefix_attention(qa, ka, va, P, G, L).backward(dout)
    qb, kb, vb = (t.clone().float().requires_grad_(True) for t in (q, k, v))
    oc, _ = grouped_prefix_causal_attention_reference(
        qb[P:].reshape(G, L, hq, 128), kb[:P], vb[:P], kb[P:].reshape(G, L, hkv, 128), vb[P:].reshape(G, L, hkv, 128)
    )
    op = torch.nn.functional.scaled_dot_product_attention(
        qb[:P].transpose(0, 1), kb[:P].transpose(0, 1).repeat_interleave(hq // hkv, 0),
        vb[:P].transpose(0, 1).repeat_interleave(hq // hkv, 0), is_causal=True,
    ).transpose(0, 1)
    torch.cat([op, oc.reshape(G * L, hq, 128)]).backward(dout.float())
    for got, want in ((qa.grad, qb.grad), (ka.grad, kb.grad), (va.grad, vb.grad)):
        scale = want.abs().max().item()
        assert (got.float() - want).abs().max().item() / scale < 3e-2


@pytest.mark.parametrize("chunk", [192, 256])
def test_overlapping_key_ranges_match_full_causal_attention(chunk):
    """Context-parallel style layout on one GPU: four query chunks in zig-zag order, each seeing the keys
    before it without a mask and its own keys causally.  The prefix of one chunk overlaps other chunks'
    self ranges, which the dK/dV work lists must cut into key tiles written exactly once."""
    from rl_engine.kernels.ops.sm100.attention import FlashAttentionSM100Op, make_layout, packed_attention

    hq, hkv, s = 4, 2, 4 * chunk
    order = [0, 3, 1, 2]  # query chunks as two zig-zag shards laid end to end
    q, k, v, do = _rand((s, hq, 128), 1), _rand((s, hkv, 128), 2), _rand((s, hkv, 128), 3), _rand((s, hq, 128), 4)
    rows = [(i * chunk, chunk, 0, cid * chunk, cid * chunk, chunk) for i, cid in enumerate(order)]
    layout = make_layout(rows, True, DEV)
    perm = torch.cat([torch.arange(c * chunk, (c + 1) * chunk, device=DEV) for c in order])
    qs = q[perm].clone().requires_grad_(True)
    ks, vs = k.clone().requires_grad_(True), v.clone().requires_grad_(True)
    out = packed_attention(qs, ks, vs, layout)
    out.backward(do[perm])
    qf, kf, vf = (t.clone().requires_grad_(True) for t in (q, k, v))
    ref = FlashAttentionSM100Op()(qf[None], kf[None], vf[None], causal=True)[0]
    ref.backward(do)
    assert torch.allclose(out.float(), ref[perm].float(), atol=2e-2, rtol=2e-2)
    for got, want in ((qs.grad, qf.grad[perm]), (ks.grad, kf.grad), (vs.grad, vf.grad)):
        scale = want.float().abs().max()
        assert (got.float() - want.float()).abs().max() / scale < 2e-2
    # and against fp32 PyTorch for the key gradients
    qd, kd, vd = (t.detach().float().requires_grad_(True) for t in (q, k, v))
    rep = hq // hkv
    sc = torch.einsum("qhd,khd->hqk", qd, kd.repeat_interleave(rep, 1)) / math.sqrt(128)
    sc = sc.masked_fill(~torch.ones(s, s, dtype=torch.bool, device=DEV).tril(), float("-inf"))
    o = torch.einsum("hqk,khd->qhd", torch.softmax(sc, -1), vd.repeat_interleave(rep, 1))
    o.backward(do.float())
    for got, want in ((ks.grad, kd.grad), (vs.grad, vd.grad)):
        assert (got.float() - want).abs().max() / want.abs().max() < 3e-2
