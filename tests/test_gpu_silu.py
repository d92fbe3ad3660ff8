"""SiLU-and-Mul kernel vs the CPU oracle, the golden vectors and torch's own CUDA arithmetic.

Mirrors the cases of the reference's tests/test_activation.py: vector body and tails, every
16-byte alignment pair, special values, all 65536 gate bit patterns, stream and graph replay.
"""

import math

import pytest
import torch
import torch.nn.functional as F

import vllm_rlt_b200 as rlt
from oracle import oracle

pytestmark = pytest.mark.gpu
DTYPES = [torch.float32, torch.float16, torch.bfloat16]


def bits(t):
    return t.view(torch.int32 if t.dtype == torch.float32 else torch.int16)


def torch_reference(gate, up):
    return F.silu(gate) * up


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("shape", [(), (0, 7), (2, 0), (1,), (7,), (8,), (9,), (3, 7), (2, 3, 9), (3, 5633), (128, 5632)])
@pytest.mark.parametrize("offsets", [(0, 0), (1, 0), (0, 1), (1, 1)])
def test_vectors_tails_and_storage_offsets(dtype, shape, offsets):
    count = math.prod(shape)
    gate = (torch.randn(count + offsets[0], device="cuda") * 3).to(dtype)[offsets[0]:].view(shape)
    up = torch.randn(count + offsets[1], device="cuda").to(dtype)[offsets[1]:].view(shape)
    gate_before, up_before = gate.clone(), up.clone()
    out = rlt.silu_and_mul(gate, up)
    assert out.shape == gate.shape and out.dtype == dtype and out.device == gate.device
    # bit-exact with torch's CUDA arithmetic, as the reference kernel is
    assert torch.equal(bits(out), bits(torch_reference(gate, up)))
    assert torch.equal(bits(gate), bits(gate_before)) and torch.equal(bits(up), bits(up_before))
    if count:
        assert out.data_ptr() not in (gate.data_ptr(), up.data_ptr())
        want = oracle.silu_and_mul(gate.cpu(), up.cpu())
        if dtype == torch.float32:
            torch.testing.assert_close(out.cpu(), want, rtol=1e-5, atol=1e-30)
        else:  # at most one unit in the last place where the fp32 exp differs by an ulp
            diff = (bits(out.cpu()).int() - bits(want).int()).abs()
            assert int(diff.max()) <= 1 and float((diff != 0).float().mean()) < 2e-3


def test_known_values_and_golden_vectors(golden):
    cases = golden("silu.pt")
    known = cases[0]
    out = rlt.silu_and_mul(known["gate"].cuda(), known["up"].cuda())
    torch.testing.assert_close(out.cpu(), known["known"])
    for case in cases:
        got = rlt.silu_and_mul(case["gate"].cuda(), case["up"].cuda()).cpu()
        want = case["out"]
        if want.dtype == torch.float32:
            torch.testing.assert_close(got, want, rtol=1e-5, atol=1e-30, equal_nan=True)
        else:
            nan = torch.isnan(want)
            assert torch.equal(torch.isnan(got), nan)
            diff = (bits(got)[~nan].int() - bits(want)[~nan].int()).abs()
            assert int(diff.max()) <= 1


@pytest.mark.parametrize("dtype", DTYPES)
def test_all_alignment_pairs_match_aligned_path(dtype):
    elements = 16 // torch.empty((), dtype=dtype).element_size()
    counts = [*range(2 * elements + 2), 17 * elements - 1, 17 * elements + 1]
    generator = torch.Generator(device="cuda").manual_seed(42)
    for count in counts:
        for gate_offset in range(elements):
            for up_offset in range(0, elements, max(1, elements // 4)):
                gate = torch.randn(count + gate_offset, device="cuda", generator=generator).to(dtype)[gate_offset:]
                up = torch.randn(count + up_offset, device="cuda", generator=generator).to(dtype)[up_offset:]
                expected = rlt.silu_and_mul(gate.clone(), up.clone())
                actual = rlt.silu_and_mul(gate, up)
                assert torch.equal(bits(actual), bits(expected)), (dtype, count, gate_offset, up_offset)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("offsets", [(0, 0), (1, 3)])
def test_special_values_and_underflow(dtype, offsets):
    info = torch.finfo(dtype)
    values = [float("nan"), float("inf"), -float("inf"), -100, -12, -1, -0.0, 0.0, 1, 12, 100,
              info.tiny, info.tiny / 128, info.max]
    gate, up = torch.meshgrid(torch.tensor(values, device="cuda", dtype=dtype),
                              torch.tensor(values, device="cuda", dtype=dtype), indexing="ij")
    gate, up = gate.contiguous(), up.contiguous()
    if offsets != (0, 0):
        count = gate.numel()
        shifted_gate = torch.empty(count + offsets[0], device="cuda", dtype=dtype)[offsets[0]:]
        shifted_up = torch.empty(count + offsets[1], device="cuda", dtype=dtype)[offsets[1]:]
        shifted_gate.copy_(gate.flatten())
        shifted_up.copy_(up.flatten())
        gate, up = shifted_gate.view(gate.shape), shifted_up.view(up.shape)
    torch.testing.assert_close(rlt.silu_and_mul(gate, up), torch_reference(gate, up), rtol=0, atol=0,
                               equal_nan=True)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("offsets", [(0, 0), (1, 3)])
def test_low_precision_storage_patterns(dtype, offsets):
    values = torch.arange(65536, device="cuda", dtype=torch.int32).to(torch.int16).view(dtype)
    info = torch.finfo(dtype)
    subnormal = info.tiny / (1024 if dtype == torch.float16 else 128)
    factors = torch.tensor([0.0, -0.0, 1.0, -1.0, 0.5, -0.5, 2.0, -2.0, info.tiny, subnormal, info.max,
                            -info.max, float("inf"), -float("inf"), float("nan")], device="cuda", dtype=dtype)
    count = values.numel() * factors.numel()
    gate = torch.empty(count + offsets[0], device="cuda", dtype=dtype)[offsets[0]:]
    up = torch.empty(count + offsets[1], device="cuda", dtype=dtype)[offsets[1]:]
    gate.copy_(values.repeat(factors.numel()))
    up.copy_(factors.repeat_interleave(values.numel()))
    actual = rlt.silu_and_mul(gate, up)
    expected = torch_reference(gate, up)
    torch.testing.assert_close(actual, expected, rtol=0, atol=0, equal_nan=True)
    valid = ~torch.isnan(expected)
    assert torch.equal(bits(actual)[valid], bits(expected)[valid])


def test_rejects_noncontiguous_and_autograd():
    gate, up = torch.randn(2, 14, device="cuda").chunk(2, dim=-1)
    with pytest.raises(RuntimeError, match="contiguous inputs"):
        rlt.silu_and_mul(gate, up)
    gate = torch.randn(16, device="cuda", requires_grad=True)
    up = torch.randn_like(gate)
    with pytest.raises(RuntimeError, match="inference-only"):
        rlt.silu_and_mul(gate, up)
    with torch.no_grad():
        out = rlt.silu_and_mul(gate, up)
        assert torch.equal(out, torch_reference(gate, up)) and not out.requires_grad


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("offsets", [(0, 0), (1, 3)])
def test_current_stream_and_graph_replay(dtype, offsets):
    count = 128 * 5632 + 3
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        gate = torch.randn(count + offsets[0], device="cuda").to(dtype)[offsets[0]:]
        up = torch.randn(count + offsets[1], device="cuda").to(dtype)[offsets[1]:]
        for _ in range(3):
            rlt.silu_and_mul(gate, up)
    stream.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=stream):
        out = rlt.silu_and_mul(gate, up)
    gate.fill_(3)
    up.fill_(2)
    graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(out, torch_reference(gate, up))


def test_torch_op_registration_dispatches_cuda_to_the_kernel():
    rlt.register_torch_op("vllm_rlt_b200_test")
    gate = torch.randn(3, 5632, device="cuda", dtype=torch.bfloat16)
    up = torch.randn_like(gate)
    out = torch.ops.vllm_rlt_b200_test.silu_and_mul(gate, up)
    assert torch.equal(out, torch_reference(gate, up))


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("rows,cols,pad", [(128, 5632, 0), (640, 5632, 0), (7, 40, 0), (5, 33, 0), (3, 24, 8), (1, 1, 0)])
def test_packed_form_reads_the_two_halves_of_one_projection_in_place(dtype, rows, cols, pad):
    # gate and up side by side in one [rows, 2 * cols] tensor (optionally a column slice of a wider one, so
    # the row stride exceeds 2 * cols); bit-identical to the two-tensor op and to F.silu(gate) * up
    g = torch.Generator().manual_seed(rows * 31 + cols)
    wide = (torch.randn(rows, 2 * cols + pad, generator=g) * 3).to(dtype).cuda()
    packed = wide[:, : 2 * cols]
    gate, up = packed[:, :cols].contiguous(), packed[:, cols:].contiguous()
    got = rlt.silu_and_mul_packed(packed)
    assert got.shape == (rows, cols) and got.is_contiguous()
    assert torch.equal(got, rlt.silu_and_mul(gate, up))
    assert torch.equal(got, torch.nn.functional.silu(gate) * up)
    with pytest.raises(ValueError):
        rlt.silu_and_mul_packed(wide[:, :3] if cols != 1 else wide[:, :1])
    assert rlt.silu_and_mul_packed(packed[:0]).shape == (0, cols)
