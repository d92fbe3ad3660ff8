"""Fused RoPE + KV write and sandwich RMSNorm vs the reference's outputs and the CPU oracle."""

import pytest
import torch

import vllm_rlt_b200 as rlt
from oracle import oracle

pytestmark = pytest.mark.gpu

ULP = {torch.float32: 2.0 ** -23, torch.float16: 2.0 ** -10, torch.bfloat16: 2.0 ** -7}


def close_to_last_place(got, want, dtype, exact_fraction=0.99):
    """Agreement to one unit in the last place of `dtype`, and exact almost everywhere."""
    got, want = got.float().cpu(), want.float().cpu()
    # the residual add cancels, so the last place is that of the operands, not of the sum
    torch.testing.assert_close(got, want, rtol=2 * ULP[dtype], atol=2 * ULP[dtype] * float(want.abs().max()))
    if dtype != torch.float32:   # a last-place difference of the fp32 scale rarely survives the rounding
        assert float((got == want).float().mean()) >= exact_fraction


def test_rope_of_the_reference_bit_for_bit(golden):
    for case in golden("layers.pt")["rope"]:
        q, k = case["q"].cuda(), case["k"].cuda()
        rows, kv_heads, dim = k.shape
        v = torch.randn_like(k)
        key_cache = torch.zeros(rows + 2, 4, kv_heads, dim, dtype=q.dtype, device="cuda")
        value_cache = torch.zeros_like(key_cache)
        blocks = torch.arange(rows, device="cuda") + 1
        offsets = torch.arange(rows, device="cuda") % 4
        q_rot = rlt.rope_kv_write(q, k, v, case["cos"].cuda(), case["sin"].cuda(), key_cache, value_cache, blocks,
                                  offsets)
        assert torch.equal(q_rot.cpu(), case["q_rot"])
        assert torch.equal(key_cache[blocks, offsets].cpu(), case["k_rot"])
        assert torch.equal(value_cache[blocks, offsets], v)
        assert not key_cache[0].any() and not key_cache[-1].any()


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32, torch.float16])
@pytest.mark.parametrize("q_heads,kv_heads,dim", [(16, 16, 128), (8, 2, 64), (3, 1, 6)])
def test_rope_kv_write_matches_oracle_on_strided_fused_projections(dtype, q_heads, kv_heads, dim):
    g = torch.Generator().manual_seed(dim)
    rows, layers, block = 45, 3, 16
    fused = torch.randn(rows, (q_heads + 2 * kv_heads) * dim + 8, generator=g).to(dtype)   # one QKV projection
    q = fused[:, :q_heads * dim].view(rows, q_heads, dim)
    k = fused[:, q_heads * dim:(q_heads + kv_heads) * dim].view(rows, kv_heads, dim)
    v = fused[:, (q_heads + kv_heads) * dim:(q_heads + 2 * kv_heads) * dim].view(rows, kv_heads, dim)
    positions = torch.randint(0, 30000, (rows,), generator=g)
    inv_freq = 1.0 / (10000.0 ** (torch.arange(0, dim, 2).float() / dim))
    angles = positions.float()[:, None] * inv_freq
    angles = torch.cat((angles, angles), -1)
    cos, sin = angles.cos().to(dtype), angles.sin().to(dtype)
    pool_k = torch.randn(7, layers, block, kv_heads, dim, generator=g).to(dtype)            # layer-strided views
    pool_v = torch.randn(7, layers, block, kv_heads, dim, generator=g).to(dtype)
    slots = torch.randperm(7 * block, generator=g)[:rows]
    blocks, offsets = slots // block, slots % block
    mask = torch.rand(rows, generator=g) > 0.2
    active = torch.tensor(40, dtype=torch.int32)
    want_k, want_v = pool_k.clone(), pool_v.clone()
    want_q = oracle.rope_kv_write(q, k, v, cos, sin, want_k[:, 1], want_v[:, 1], blocks, offsets, mask, active)
    got_k, got_v, gpu_fused = pool_k.cuda(), pool_v.cuda(), fused.cuda()
    got_q = rlt.rope_kv_write(gpu_fused[:, :q_heads * dim].view(rows, q_heads, dim),
                              gpu_fused[:, q_heads * dim:(q_heads + kv_heads) * dim].view(rows, kv_heads, dim),
                              gpu_fused[:, (q_heads + kv_heads) * dim:(q_heads + 2 * kv_heads) * dim].view(
                                  rows, kv_heads, dim),
                              cos.cuda(), sin.cuda(), got_k[:, 1], got_v[:, 1], blocks.cuda(), offsets.cuda(),
                              mask.cuda(), active.cuda())
    assert torch.equal(got_q.cpu(), want_q)
    assert torch.equal(got_k.cpu(), want_k) and torch.equal(got_v.cpu(), want_v)
    # masked and inactive rows wrote nothing; the other layers of the pool are untouched
    skipped = (~mask) | (torch.arange(rows) >= 40)
    assert torch.equal(got_k.cpu()[blocks[skipped], 1, offsets[skipped]], pool_k[blocks[skipped], 1, offsets[skipped]])
    assert torch.equal(got_k.cpu()[:, 0], pool_k[:, 0]) and torch.equal(got_k.cpu()[:, 2], pool_k[:, 2])
    # and the tensor expression itself
    c, s = cos[:, None], sin[:, None]
    rotate = lambda x: torch.cat((-x[..., dim // 2:], x[..., :dim // 2]), -1)
    assert torch.equal(want_q, q * c + rotate(q) * s)


def test_rope_kv_write_never_reads_the_address_of_a_skipped_row():
    rows, heads, dim = 4, 2, 64
    q = torch.randn(rows, heads, dim, device="cuda", dtype=torch.bfloat16)
    cache = torch.zeros(2, 16, heads, dim, device="cuda", dtype=torch.bfloat16)
    value = torch.zeros_like(cache)
    blocks = torch.tensor([0, 1 << 40, -5, 1], device="cuda")          # rows 1, 2 carry garbage addresses
    offsets = torch.tensor([3, 1 << 40, 0, 99], device="cuda")         # row 3: offset outside the page
    ones = torch.ones(rows, dim, device="cuda", dtype=torch.bfloat16)
    out = rlt.rope_kv_write(q, q, q, ones, torch.zeros_like(ones), cache, value, blocks, offsets)
    assert torch.equal(out, q)
    assert torch.equal(cache[0, 3], q[0]) and int((cache != 0).any(-1).any(-1).sum()) == 1


def test_sandwich_norm_of_the_reference(golden):
    for case in golden("layers.pt")["norm"]:
        dtype = case["x"].dtype
        x, w, w2, residual = (case[n].cuda() for n in ("x", "weight", "weight2", "residual"))
        plain, _ = rlt.sandwich_norm(x, w, case["eps"])
        close_to_last_place(plain, case["plain"], dtype)
        total, following = rlt.sandwich_norm(x, w, case["eps"], residual, w2)
        close_to_last_place(total, case["total"], dtype)
        # the second norm sees a total that may differ in the last place: compare at two places
        torch.testing.assert_close(following.float().cpu(), case["following"].float(), rtol=4 * ULP[dtype],
                                   atol=4 * ULP[dtype] * float(case["following"].abs().max()))


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32, torch.float16])
@pytest.mark.parametrize("rows,hidden", [(640, 2048), (3, 100), (5, 8192)])
def test_sandwich_norm_matches_oracle(dtype, rows, hidden):
    g = torch.Generator().manual_seed(hidden)
    x = (torch.randn(rows, hidden, generator=g) * 3).to(dtype)
    x[0] = 0                                                        # a zero row stays zero (padding rows)
    residual = torch.randn(rows, hidden, generator=g).to(dtype)
    w = (1 + 0.2 * torch.randn(hidden, generator=g)).to(dtype)
    w2 = (1 + 0.2 * torch.randn(hidden, generator=g)).to(dtype)
    want_total, want_norm = oracle.sandwich_norm(x, w, 1e-6, residual, w2)
    got_total, got_norm = rlt.sandwich_norm(x.cuda(), w.cuda(), 1e-6, residual.cuda(), w2.cuda())
    # the double-precision sum of squares makes the two agree bit for bit in practice
    assert torch.equal(got_total.cpu(), want_total) and torch.equal(got_norm.cpu(), want_norm)
    want_plain, _ = oracle.sandwich_norm(x, w, 1e-6)
    got_plain, none = rlt.sandwich_norm(x.cuda(), w.cuda(), 1e-6)
    assert none is None and torch.equal(got_plain.cpu(), want_plain) and not got_plain[0].any()
    # in place on the residual stream
    stream = residual.cuda().clone()
    total, norm = rlt.sandwich_norm(x.cuda(), w.cuda(), 1e-6, stream, w2.cuda(), in_place=True)
    assert total.data_ptr() == stream.data_ptr() and torch.equal(stream.cpu(), want_total)
    assert torch.equal(norm.cpu(), want_norm)


def test_layer_kernels_validate_their_arguments():
    x = torch.randn(2, 16384, device="cuda")
    with pytest.raises(NotImplementedError, match="8192"):
        rlt.sandwich_norm(x, torch.ones(16384, device="cuda"), 1e-6)
    with pytest.raises(ValueError):
        rlt.sandwich_norm(x.t(), torch.ones(2, device="cuda"), 1e-6)
    q = torch.randn(2, 2, 7, device="cuda")
    with pytest.raises(ValueError, match="even"):
        rlt.rope_kv_write(q, q, q, q[:, 0], q[:, 0], torch.zeros(1, 4, 2, 7, device="cuda"),
                          torch.zeros(1, 4, 2, 7, device="cuda"), torch.zeros(2, dtype=torch.int64, device="cuda"),
                          torch.zeros(2, dtype=torch.int64, device="cuda"))
