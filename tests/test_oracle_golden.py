"""The CPU oracle against outputs of the reference's own code (tests/golden/*)."""

import hashlib

import numpy as np
import pytest
import torch

from conftest import rel_l2
from leankv_b200 import workloads
from oracle import pool_layout, teal as oteal, tq_exact, turboquant as otq


def test_codebook_matches_reference(golden_codebooks):
    got = otq.lloyd_max(128, 3)
    assert got["centroids"] == golden_codebooks["3"]["centroids"]
    assert got["boundaries"] == golden_codebooks["3"]["boundaries"]


def test_rotation_matches_reference(golden_rotations):
    for seed in (42, 43, 77, 105):
        Pi = otq.rotation_matrix(128, seed)
        assert hashlib.sha256(Pi.numpy().tobytes()).hexdigest() == golden_rotations[str(seed)]["sha256"]


def test_teal_config1_and_2(golden_teal):
    c1 = workloads.sparse_gemv_case()
    t = oteal.threshold_for_sparsity(c1.x, 0.4)
    assert t == float(golden_teal["c1_threshold"])
    assert oteal.n_active(c1.x, t) == int(golden_teal["c1_n_active"]) == c1.n_active
    y = oteal.sparse_linear(c1.x, c1.weight, t)
    assert torch.equal(y, torch.from_numpy(golden_teal["c1_y_fp16"]))
    c2 = workloads.swiglu_case()
    t2 = oteal.threshold_for_sparsity(c2.x, 0.4)
    assert t2 == float(golden_teal["c2_threshold"])
    y2 = oteal.swiglu(c2.x, c2.w_gate, c2.w_up, t2, t2)
    assert torch.equal(y2, torch.from_numpy(golden_teal["c2_y_fp16"]))
    y2_32 = oteal.swiglu(c2.x, c2.w_gate, c2.w_up, t2, t2, accumulate="fp32")
    assert rel_l2(y2_32, golden_teal["c2_y_fp16"]) < 1e-3


def test_teal_small_cases(golden_teal):
    for i, (n, z, s, seed) in enumerate(golden_teal["small_cases"]):
        c = workloads.sparse_gemv_case(int(n), int(z), float(s), int(seed))
        t = oteal.threshold_for_sparsity(c.x, float(s))
        assert t == float(golden_teal[f"small{i}_threshold"])
        mask = (c.x.abs() > t) if t > 0 else torch.ones_like(c.x, dtype=torch.bool)
        assert np.array_equal(mask.numpy(), golden_teal[f"small{i}_mask"])
        y32 = oteal.sparse_linear(c.x, c.weight, t, accumulate="fp32")
        assert torch.allclose(y32, torch.from_numpy(golden_teal[f"small{i}_y_fp32"]), rtol=1e-5, atol=1e-6)


def test_histogram_threshold(golden_teal):
    counts = torch.from_numpy(golden_teal["hist_counts"])
    edges = torch.from_numpy(golden_teal["hist_edges"])
    for s, want in zip(golden_teal["hist_targets"], golden_teal["hist_thresholds"]):
        assert oteal.threshold_from_histogram(counts, edges, float(s)) == pytest.approx(float(want), rel=1e-6)


def _small_kv():
    return workloads.kv_case(batch=2, n_q_heads=8, n_kv_heads=2, context=70, seed=3)


def test_quantize_torch_restatement_is_bit_identical(golden_tq):
    kv = _small_kv()
    bounds = torch.from_numpy(golden_tq["decision_boundaries"])
    for name, seed, x in (("k", 42, kv.k), ("v", 43, kv.v)):
        Pi = otq.rotation_matrix(128, seed)
        packed, norms, _, y = otq.quantize(x.float(), Pi, bounds, 3)
        assert np.array_equal(packed.numpy(), golden_tq[f"{name}_indices"])
        assert np.array_equal(norms.numpy(), golden_tq[f"{name}_norms"])
        assert np.array_equal(y.numpy(), golden_tq[f"{name}_rotated"])
        deq = otq.dequantize(packed, norms, Pi, torch.from_numpy(golden_tq["centroids"]), 3, 128)
        assert np.array_equal(deq.numpy(), golden_tq[f"{name}_dequant"])


def test_exact_order_oracle_vs_reference_codes(golden_tq):
    """The fixed-order C restatement may differ from the reference (BLAS order) only where the
    rotated coordinate is within rounding distance of a decision boundary."""
    kv = _small_kv()
    bounds = golden_tq["decision_boundaries"]
    n_total = n_diff = 0
    for name, seed, x in (("k", 42, kv.k), ("v", 43, kv.v)):
        Pi = otq.rotation_matrix(128, seed).numpy()
        codes, norms, y, margin = tq_exact.quantize(x.float().numpy().reshape(-1, 128), Pi, bounds)
        ref_codes = pool_layout.nibbles_to_codes(golden_tq[f"{name}_indices"]).reshape(-1, 128)
        ref_norms = golden_tq[f"{name}_norms"].reshape(-1)
        diff = codes != ref_codes
        n_total += codes.size
        n_diff += int(diff.sum())
        # a mismatch is legitimate only as a near-tie: |y - b| <= 4 ulp of y
        assert np.all(margin[diff] <= 4 * np.spacing(np.abs(y[diff]).astype(np.float32)))
        # norms: correctly rounded here, fp32-accumulated in the reference: <= 2 ulp apart
        assert np.all(np.abs(norms - ref_norms) <= 2 * np.spacing(ref_norms))
        assert np.max(np.abs(y - golden_tq[f"{name}_rotated"].reshape(-1, 128))) < 2e-7
    assert n_diff <= max(1, n_total // 100000)


def test_exact_dequantize_vs_reference(golden_tq):
    kv = _small_kv()
    Pi = otq.rotation_matrix(128, 42).numpy()
    codes = pool_layout.nibbles_to_codes(golden_tq["k_indices"]).reshape(-1, 128)
    deq = tq_exact.dequantize(codes, golden_tq["k_norms"], Pi, golden_tq["centroids"])
    assert rel_l2(deq, golden_tq["k_dequant"].reshape(-1, 128)) < 1e-6


def test_attention_restatement(golden_tq):
    kv = _small_kv()
    k_hat = torch.from_numpy(golden_tq["k_dequant_fp16norm_half"])
    v_hat = torch.from_numpy(golden_tq["v_dequant_fp16norm_half"])
    out = otq.kv_attention(kv.q, k_hat, v_hat, 128 ** -0.5, lengths=golden_tq["attn_lengths"].tolist())
    assert torch.allclose(out, torch.from_numpy(golden_tq["attn_out"]), rtol=1e-5, atol=1e-6)


def test_other_bit_widths_and_packing(golden_tq, golden_codebooks):
    kv = _small_kv()
    xs = kv.k[0, 0, :9].float()
    for bits in (1, 2, 4):
        cb = golden_codebooks[str(bits)]
        bounds = torch.tensor(cb["boundaries"][1:-1], dtype=torch.float32)
        cents = torch.tensor(cb["centroids"], dtype=torch.float32)
        Pi = otq.rotation_matrix(128, 7)
        packed, norms, _, _ = otq.quantize(xs, Pi, bounds, bits)
        assert np.array_equal(packed.numpy(), golden_tq[f"b{bits}_indices"])
        deq = otq.dequantize(packed, norms, Pi, cents, bits, 128)
        assert np.array_equal(deq.numpy(), golden_tq[f"b{bits}_dequant"])
    for bits in (1, 2, 3, 4, 6):
        codes = torch.from_numpy(golden_tq[f"pack_b{bits}_codes"])
        packed = otq.pack(codes, bits)
        assert np.array_equal(packed.numpy(), golden_tq[f"pack_b{bits}_packed"])
        assert torch.equal(otq.unpack(packed, bits, 13), codes)


def test_pool_layout_round_trip():
    rng = np.random.default_rng(0)
    for which in (0, 1):
        codes = rng.integers(0, 8, size=(16, 128), dtype=np.uint8)
        norms = rng.random(16).astype(np.float16).astype(np.float32)
        chunk = pool_layout.encode_chunk(codes, norms, which)
        got_codes, got_norms = pool_layout.decode_chunk(chunk, which)
        assert np.array_equal(got_codes, codes)
        assert np.array_equal(got_norms, norms)
        # every bit of the 768 code bytes is used exactly once: all-7 codes fill the words
        full = pool_layout.encode_chunk(np.full((16, 128), 7, np.uint8), norms, which)
        assert np.all(full[:768] == 0xFF)
