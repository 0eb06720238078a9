"""Row-wise e4m3 quantisation of the operator's inputs: oracle vs the reference's recorded
outputs (CPU), and the CUDA kernel (through the C ABI) vs both (GPU).  Bit-exact throughout."""

from __future__ import annotations

import sys
from pathlib import Path

import numpy as np
import pytest
import torch

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))
from oracle import oracle  # noqa: E402

from fusedindextopk_b200 import inputs as host_inputs  # noqa: E402

_DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def _golden_case(entry):
    dtype = _DTYPES[entry["dtype"]]
    raw = torch.frombuffer(bytearray.fromhex(entry["source_hex"]), dtype=torch.uint8)
    source = raw.view(dtype).reshape(entry["rows"], 128).clone()
    values = np.frombuffer(bytes.fromhex(entry["values_hex"]), dtype=np.uint8).reshape(entry["rows"], 128)
    scales = np.frombuffer(bytes.fromhex(entry["scales_hex"]), dtype=np.uint32)
    return source, values, scales


def test_oracle_reproduces_the_reference_quantisation(golden):
    assert len(golden["quantize_index_kv"]) == 2
    for entry in golden["quantize_index_kv"]:
        source, values, scales = _golden_case(entry)
        codes, got_scales = oracle.quantize_rows_e4m3(source.float().numpy())
        assert np.array_equal(codes, values)
        assert np.array_equal(got_scales.view(np.uint32), scales)


def test_host_recipe_reproduces_the_reference_quantisation(golden):
    for entry in golden["quantize_index_kv"]:
        source, values, scales = _golden_case(entry)
        got_values, got_scales = host_inputs.quantize_rows_e4m3(source)
        assert np.array_equal(got_values.view(torch.uint8).numpy(), values)
        assert np.array_equal(got_scales.numpy().view(np.uint32), scales)


def test_encode_e4m3_known_answers():
    # ties go to the even code: 17 -> 16 (0x58), 19 -> 20 (0x5a), 2^-10 -> 0, 3*2^-10 -> 2*2^-9
    values = np.array([17.0, 19.0, 2.0 ** -10, 3 * 2.0 ** -10, 448.0, -448.0, 463.9, -0.0, 1.0625], dtype=np.float32)
    codes = oracle.encode_e4m3(values)
    assert codes.tolist() == [0x58, 0x5A, 0x00, 0x02, 0x7E, 0xFE, 0x7E, 0x80, 0x38]
    with pytest.raises(ValueError):
        oracle.encode_e4m3(np.array([464.0], dtype=np.float32))


# ----------------------------------------------------------------------------- GPU


@pytest.fixture(scope="module")
def device():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    return torch.device("cuda:0")


def _assert_bit_exact(source_cpu, values_gpu, scales_gpu):
    codes, scales = oracle.quantize_rows_e4m3(source_cpu.float().numpy().reshape(-1, 128))
    assert np.array_equal(values_gpu.view(torch.uint8).cpu().numpy().reshape(-1, 128), codes)
    if scales_gpu is not None:
        assert np.array_equal(scales_gpu.cpu().numpy().reshape(-1).view(np.uint32), scales.view(np.uint32))
    return scales


@pytest.mark.gpu
def test_kernel_reproduces_the_reference_quantisation(golden, device):
    from fusedindextopk_b200 import quantize

    for entry in golden["quantize_index_kv"]:
        source, values, scales = _golden_case(entry)
        got_values, got_scales = quantize.quantize_contiguous_index_kv(source.to(device))
        assert got_values.dtype == torch.float8_e4m3fn and got_scales.dtype == torch.float32
        assert np.array_equal(got_values.view(torch.uint8).cpu().numpy(), values)
        assert np.array_equal(got_scales.cpu().numpy().view(np.uint32), scales)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rows", [1, 31, 32, 33, 4097])
def test_kernel_matches_oracle_on_ragged_row_counts(device, dtype, rows):
    from fusedindextopk_b200 import quantize

    generator = torch.Generator().manual_seed(rows)
    source = (torch.randn((rows, 128), generator=generator)
              * torch.exp(3.0 * torch.randn((rows, 1), generator=generator))).to(dtype)
    source[0] = 0.0
    values, scales = quantize.quantize_contiguous_index_kv(source.to(device))
    _assert_bit_exact(source, values, scales)


@pytest.mark.gpu
def test_kernel_division_is_correctly_rounded_over_a_wide_dynamic_range(device):
    """One million quotients with element exponents spread over 2^-120 .. 2^0 of the row
    maximum, row maxima over 2^-30 .. 2^100, plus rows on the amax floor."""

    from fusedindextopk_b200 import quantize

    generator = torch.Generator().manual_seed(77)
    rows = 8192
    mantissa = torch.randn((rows, 128), generator=generator)
    exponent = -torch.rand((rows, 128), generator=generator) ** 4 * 120.0
    row_scale = torch.exp2(torch.rand((rows, 1), generator=generator) * 130.0 - 30.0)
    source = (mantissa * torch.exp2(exponent) * row_scale).float()
    source[:64] = mantissa[:64] * 1e-5          # below the amax floor: scale = 1e-4 / 448
    source[64:128] = torch.round(mantissa[64:128] * 64.0) / 64.0 * 448.0 / 4.0   # many exact code midpoints
    source[64:128, 0] = 448.0 * 2.0
    values, scales = quantize.quantize_contiguous_index_kv(source.to(device))
    _assert_bit_exact(source, values, scales)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_query_quantisation_folds_the_scale_into_the_weights(device, dtype):
    from fusedindextopk_b200 import quantize

    generator = torch.Generator().manual_seed(5)
    source = torch.randn((48, 64, 128), generator=generator).to(dtype)
    source[::7] *= 4.0
    weights = torch.randn((48, 64), generator=generator)
    q, folded = quantize.quantize_queries(source.to(device), weights.to(device))
    scales = _assert_bit_exact(source, q, None)
    expected = weights.numpy().reshape(-1) * scales
    assert np.array_equal(folded.cpu().numpy().reshape(-1).view(np.uint32), expected.astype(np.float32).view(np.uint32))


@pytest.mark.gpu
def test_full_size_query_tensor_round_trips(device):
    """c1-sized queries (262144 rows): every row's largest magnitude maps to +-448 and the
    decoded values stay within half an e4m3 step of the scaled source."""

    from fusedindextopk_b200 import quantize

    generator = torch.Generator().manual_seed(9)
    source = torch.randn((4096, 64, 128), generator=generator, dtype=torch.float32).to(torch.bfloat16)
    on_device = source.to(device)
    values, scales, _ = quantize.quantize_rows(on_device)
    decoded = values.float()
    assert bool((decoded.abs().amax(dim=-1) == 448.0).all())
    scaled = on_device.float() / scales.unsqueeze(-1)
    step = torch.maximum(torch.exp2(torch.floor(torch.log2(scaled.abs().clamp_min(2.0 ** -6))) - 3), torch.tensor(2.0 ** -9, device=device))
    assert bool(((decoded - scaled).abs() <= 0.5 * step).all())
    # a strided sample of rows against the oracle, bit for bit
    pick = torch.arange(0, 4096 * 64, 997)
    codes, oracle_scales = oracle.quantize_rows_e4m3(source.reshape(-1, 128)[pick].float().numpy())
    assert np.array_equal(values.view(torch.uint8).reshape(-1, 128)[pick.to(device)].cpu().numpy(), codes)
    assert np.array_equal(scales.reshape(-1)[pick.to(device)].cpu().numpy().view(np.uint32), oracle_scales.view(np.uint32))


@pytest.mark.gpu
def test_operator_from_activations_equals_operator_on_host_quantised_inputs(device):
    from fusedindextopk_b200 import quantize
    from fusedindextopk_b200.operator import fused_index_topk

    generator = torch.Generator().manual_seed(21)
    rows, keys = 64, 8192
    q_source = torch.randn((rows, 64, 128), generator=generator).to(torch.bfloat16)
    kv_source = (torch.randn((keys, 128), generator=generator)
                 * torch.exp(0.5 * torch.randn((keys, 1), generator=generator))).to(torch.bfloat16)
    weights = torch.randn((rows, 64), generator=generator) / 64.0
    k_start, k_end = host_inputs.causal_ranges(torch, rows, keys)
    got = quantize.fused_index_topk_from_activations(
        q_source.to(device), kv_source.to(device), weights.to(device), k_start.to(device), k_end.to(device))
    q, q_scales = host_inputs.quantize_rows_e4m3(q_source)
    kv, kv_scales = host_inputs.quantize_rows_e4m3(kv_source)
    want = fused_index_topk(q.to(device), (kv.to(device), kv_scales.to(device)),
                            (weights * q_scales).to(device), k_start.to(device), k_end.to(device))
    assert torch.equal(got.sort(dim=-1).values, want.sort(dim=-1).values)


@pytest.mark.gpu
def test_argument_errors_are_reported_not_launched(device):
    from fusedindextopk_b200 import _lib, quantize

    with pytest.raises(ValueError):
        quantize.quantize_contiguous_index_kv(torch.zeros((4, 4, 128), device=device))
    with pytest.raises(ValueError):
        quantize.quantize_rows(torch.zeros((4, 64), device=device))
    with pytest.raises(TypeError):
        quantize.quantize_rows(torch.zeros((4, 128), device=device, dtype=torch.float16))
    with pytest.raises(_lib.ItkError):
        _lib.check(_lib.load_library().itk_quantize_rows_e4m3(None, 0, None, None, None, None, 4, None))
