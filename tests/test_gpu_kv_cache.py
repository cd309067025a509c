"""The KV-cache writer kernels against the CPU oracle (itself pinned to the reference's quantiser by the golden
fixture): bytes and indices bit-exact."""
import numpy as np
import pytest
import torch

import flashmla_b200
from flashmla_b200 import workloads as wl
from oracle import quant
from helpers import bf16, load_golden
from gpu_utils import DEV

pytestmark = pytest.mark.gpu


def edge_case_kv(nb, page, seed):
    gen = torch.Generator().manual_seed(seed)
    kv = torch.randn((nb, page, 1, 576), generator=gen)
    kv[0, 0] *= 1e-6                 # below the 1e-4 floor of the scale rule
    kv[1, 3, 0, :128] = 0.0          # an all-zero tile
    kv[2] *= 37.0
    kv[3, :, :, 128:256] *= 448.0
    kv[4, :, :, :32] = 448.0 * 2.0 ** -3    # amax / 448 exactly a power of two
    kv[5] *= 1e4
    return kv.to(torch.bfloat16)


@pytest.mark.parametrize("layout", [wl.LAYOUT_V32, wl.LAYOUT_MXFP8])
@pytest.mark.parametrize("row_pad", [0, 1])
def test_quantiser_is_byte_exact(layout, row_pad):
    kv = edge_case_kv(9, 13, seed=7)
    ref = quant.quantize_rows(kv, layout)
    got = flashmla_b200.quantize_k_cache(kv.to(DEV), layout, row_pad=row_pad)
    assert got.stride(0) == (13 + row_pad) * 656
    assert torch.equal(got.cpu(), ref), "quantised rows differ from the oracle"
    # and what the attention kernels read back is what the oracle dequantises
    assert torch.equal(quant.dequantize_rows(got.cpu().contiguous(), layout), quant.dequantize_rows(ref, layout))


def test_quantiser_matches_the_reference_fixture():
    g = load_golden("quant_v32")
    kv = bf16(g["kv"])
    got = flashmla_b200.quantize_k_cache(kv.to(DEV))
    assert np.array_equal(got.cpu().numpy().reshape(g["rows"].shape), g["rows"])


def test_model1_quantiser_matches_the_reference_fixture_and_the_oracle():
    """The d_qk = 512 block-wise format (tests/quant.py:55-75 of the reference)."""
    g = load_golden("quant_model1")
    got = flashmla_b200.quantize_k_cache(bf16(g["kv"]).to(DEV))          # 512 values per row: "model1" by default
    assert tuple(got.shape) == (5, 16, 1, 584) and got.stride(0) % 576 == 0
    assert np.array_equal(got.cpu().numpy(), g["rows"])
    gen = torch.Generator().manual_seed(8)
    kv = torch.randn((7, 64, 1, 512), generator=gen)
    kv[2] *= 1e3
    kv[3, :, :, :64] = 0.0
    kv = kv.to(torch.bfloat16)
    assert torch.equal(flashmla_b200.quantize_k_cache(kv.to(DEV), wl.LAYOUT_MODEL1).cpu(), quant.quantize_rows(kv, quant.LAYOUT_MODEL1))


def test_cache_indices_are_bit_exact():
    g = load_golden("quant_v32")
    pos, table = torch.from_numpy(g["positions"]), torch.from_numpy(g["block_table"])
    got = flashmla_b200.abs_indices2indices_in_kvcache(pos.to(DEV), table.to(DEV), int(g["page"]))
    assert np.array_equal(got.cpu().numpy(), g["cache_rows"])
    gen = torch.Generator().manual_seed(3)
    table = torch.randperm(40 * 17, generator=gen).to(torch.int32).view(17, 40)
    pos = torch.randint(-1, 40 * 64, (17, 3, 257), generator=gen, dtype=torch.int32)
    got = flashmla_b200.abs_indices2indices_in_kvcache(pos.to(DEV), table.to(DEV), 64)
    assert torch.equal(got.cpu(), quant.abs_to_cache_indices(pos, table, 64))


def test_full_size_pool_roundtrip():
    """A decode-benchmark-sized pool (1.2 GB of bf16 rows): every 997th block against the oracle."""
    gen = torch.Generator(device=DEV).manual_seed(5)
    kv = torch.randn((16384, 64, 1, 576), generator=gen, device=DEV, dtype=torch.float32).to(torch.bfloat16)
    rows = flashmla_b200.quantize_k_cache(kv)
    sel = torch.arange(0, 16384, 997, device=DEV)
    assert torch.equal(rows[sel].cpu(), quant.quantize_rows(kv[sel].cpu(), wl.LAYOUT_V32))
