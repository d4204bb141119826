"""Host-side logic and the C ABI surface; nothing here launches a kernel."""

import ctypes
import hashlib
import json
import os
import re

import numpy as np
import pytest
import torch

from conftest import ROOT
from leankv_b200 import _native
from leankv_b200.teal import patching, sparse_fns
from leankv_b200.turboquant import codebook, quantizer, rotation
from oracle import teal as oteal


def _declared_functions():
    text = open(os.path.join(ROOT, "include", "leankv_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(leankv_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    lib = _native.lib()
    names = _declared_functions()
    assert len(names) >= 20
    for name in names:
        assert hasattr(lib, name), f"{name} declared in the header but not exported"
        assert name in _native.SIGNATURES, f"{name} has no ctypes signature"
    assert sorted(_native.SIGNATURES) == names
    assert lib.leankv_abi_version() == 2
    assert b"workspace" in lib.leankv_strerror(-3)


def _no_device_for_made_up_pointers():
    """The validation tests pass made-up addresses and rely on every call being refused before a
    launch. Where a GPU is visible a regression of a check would launch a kernel on those addresses,
    so the tests only run on machines without one (the build container)."""
    import torch

    if torch.cuda.is_available():
        pytest.skip("made-up pointers are only passed where no kernel could be launched")


def test_argument_validation_returns_codes_before_any_launch():
    _no_device_for_made_up_pointers()
    lib = _native.lib()
    fake = 0x10000   # never dereferenced: validation fails first
    # N not a multiple of 8
    assert lib.leankv_sparse_gemv_f16(fake, fake, fake, 12, 64, 0.1, None, None, None, 0, None, None) == -2
    # null pointers / bad sizes
    assert lib.leankv_sparse_gemv_f16(None, fake, fake, 16, 64, 0.1, None, None, None, 0, None, None) == -1
    assert lib.leankv_sparse_gemv_f16(fake, fake, fake, 16, 0, 0.1, None, None, None, 0, None, None) == -1
    # split-K needs a workspace
    assert lib.leankv_sparse_gemv_f16(fake, fake, fake, 4096, 4096, 0.1, None, None, None, 0, None, None) == -3
    need = lib.leankv_sparse_gemv_workspace_bytes(4096, 4096)
    assert need > 0
    assert lib.leankv_sparse_gemv_f16(fake, fake, fake, 4096, 4096, 0.1, None, None, fake, need - 1, None, None) == -3
    # segments: boundary not on a 256-column slice
    segs = _native.Segments()
    segs.n_segments = 2
    segs.seg_end[0], segs.seg_end[1] = 100 * 8, 4096
    assert lib.leankv_sparse_gemv_seg_f16(fake, fake, fake, 4096, 64, ctypes.byref(segs), None, None,
                                          fake, 1 << 30, None, None) == -2
    segs.seg_end[0], segs.seg_end[1] = 1024, 2048   # last end != N
    assert lib.leankv_sparse_gemv_seg_f16(fake, fake, fake, 4096, 64, ctypes.byref(segs), None, None,
                                          fake, 1 << 30, None, None) == -1
    # TurboQuant: unsupported shapes
    assert lib.leankv_tq_quantize(fake, 0, 4, 64, 3, fake, fake, fake, fake, None) == -5
    assert lib.leankv_tq_quantize(fake, 0, 4, 128, 5, fake, fake, fake, fake, None) == -5
    assert lib.leankv_tq_quantize(fake, 0, 0, 128, 3, fake, fake, fake, fake, None) == 0   # empty input
    assert lib.leankv_tq_packed_len(128, 3) == 64
    assert lib.leankv_tq_packed_len(128, 2) == 32
    assert lib.leankv_tq_packed_len(128, 1) == 16
    assert lib.leankv_tq_pool_bytes(10, 8) == 10 * 2 * 8 * 800
    # attention: only GQA-4
    assert lib.leankv_tq_decode_attn(fake, fake, 1, 32, 32, fake, 4, fake, fake, fake, 4, fake, fake,
                                     fake, 0.1, fake, 1 << 30, None) == -5
    assert lib.leankv_tq_decode_attn(fake, fake, 1, 32, 8, fake, 4, fake, fake, fake, 4, fake, fake,
                                     fake, 0.1, fake, 16, None) == -3
    assert lib.leankv_tq_decode_attn(fake, fake, 0, 32, 8, fake, 4, fake, fake, fake, 4, fake, fake,
                                     fake, 0.1, fake, 16, None) == 0    # empty batch
    # unknown flag bits of the pre-rotated entry are refused
    assert lib.leankv_tq_decode_attn_rotated(fake, fake, 1, 32, 8, fake, 4, fake, fake, fake, 4, fake, fake, 0.1,
                                             fake, 1 << 30, 2, None) == -1
    # RMSNorm fused in: the output may not overlap the input row (other CTAs still read it)
    segs1 = _native.Segments()
    segs1.n_segments, segs1.seg_end[0], segs1.threshold[0] = 1, 4096, 0.1
    assert lib.leankv_sparse_gemv_rmsnorm_f16(fake * 16, fake, fake * 2, 1e-5, fake, 4096, 4096, ctypes.byref(segs1),
                                              None, fake * 4, 1 << 30, None, None) == -1
    assert lib.leankv_sparse_swiglu_rmsnorm_f16(fake * 16, fake * 32, fake, fake * 2, 1e-5, fake + 4096, 4096, 4096,
                                                0.1, 0.1, fake * 4, 1 << 30, None, None) == -1


def test_workspace_sizes_are_modest():
    lib = _native.lib()
    for n, z in ((4096, 14336), (6144, 4096), (14336, 4096), (32768, 4096), (1024, 4096)):
        assert 0 < lib.leankv_sparse_gemv_workspace_bytes(n, z) < 16 << 20
    assert lib.leankv_sparse_swiglu_workspace_bytes(14336, 4096) < 16 << 20
    assert lib.leankv_tq_decode_attn_workspace_bytes(16, 32, 8, 256) < 16 << 20


def test_no_cpu_fallback():
    x = torch.randn(4, 128)
    q = quantizer.TurboQuantMSE(128, 3, device="cpu")
    with pytest.raises(RuntimeError, match="CUDA"):
        q.quantize(x)
    from leankv_b200.teal.kernels.sparse_gemv import sparse_gemv
    with pytest.raises(RuntimeError, match="CUDA"):
        sparse_gemv(torch.randn(1, 1, 16).half(), torch.randn(8, 16).half(), 0.1)
    from leankv_b200.turboquant.cache import TurboQuantCache
    c = TurboQuantCache(num_layers=1, device="cpu")
    with pytest.raises(RuntimeError, match="CUDA"):
        c.update(torch.randn(1, 2, 3, 128).half(), torch.randn(1, 2, 3, 128).half(), 0)


def test_codebooks_and_rotations_match_reference(golden_codebooks, golden_rotations):
    for bits in (1, 2, 3, 4):
        cb = codebook.get_codebook(128, bits)
        assert cb["centroids"] == golden_codebooks[str(bits)]["centroids"]
        assert cb["boundaries"] == golden_codebooks[str(bits)]["boundaries"]
    cents, bounds = codebook.get_codebook_tensors(128, 3, "cpu")
    assert cents.shape == (8,) and bounds.shape == (9,)
    for seed in range(42, 106):
        Pi = rotation.generate_rotation_matrix(128, "cpu", torch.float32, seed)
        assert hashlib.sha256(Pi.numpy().tobytes()).hexdigest() == golden_rotations[str(seed)]["sha256"]
    q = quantizer.TurboQuantMSE(128, 3, device="cpu", seed=42)
    assert q.decision_boundaries.shape == (7,)
    assert torch.equal(q.decision_boundaries, bounds[1:-1])


def test_pack_unpack_match_reference(golden_tq):
    for bits in (1, 2, 3, 4, 6):
        codes = torch.from_numpy(golden_tq[f"pack_b{bits}_codes"])
        packed = quantizer._pack_indices(codes, bits)
        assert packed.dtype == torch.uint8
        assert np.array_equal(packed.numpy(), golden_tq[f"pack_b{bits}_packed"])
        assert torch.equal(quantizer._unpack_indices(packed, bits, 13), codes)


def test_thresholds_match_reference(golden_teal):
    from leankv_b200 import workloads

    c1 = workloads.sparse_gemv_case()
    assert c1.threshold == float(golden_teal["c1_threshold"])
    assert c1.n_active == int(golden_teal["c1_n_active"])
    assert sparse_fns.compute_threshold_for_sparsity(c1.x, 0.0) == 0.0
    assert sparse_fns.compute_threshold_for_sparsity(c1.x, 1.0) == c1.x.abs().max().item()
    counts = torch.from_numpy(golden_teal["hist_counts"])
    edges = torch.from_numpy(golden_teal["hist_edges"])
    for s, want in zip(golden_teal["hist_targets"], golden_teal["hist_thresholds"]):
        got = sparse_fns.compute_threshold_from_histogram(counts, edges, float(s))
        assert got == pytest.approx(float(want), rel=1e-6)


def test_sparsify_fn_matches_oracle():
    x = torch.randn(3, 7, 64).half()
    sf = sparse_fns.SparsifyFn(0.5)
    y = sf(x)
    assert torch.equal(y, oteal.sparsify(x, 0.5))
    assert sf.last_sparsity == pytest.approx(1.0 - (x.abs() > 0.5).float().mean().item())
    assert sparse_fns.SparsifyFn(0.0)(x) is x
    assert sparse_fns.SparsifyFn(0.5, enabled=False)(x) is x


def _tiny_model():
    from transformers import MistralConfig, MistralForCausalLM

    torch.manual_seed(0)
    cfg = MistralConfig(vocab_size=100, hidden_size=64, intermediate_size=128, num_hidden_layers=2,
                        num_attention_heads=4, num_key_value_heads=2, head_dim=16,
                        max_position_embeddings=64)
    return MistralForCausalLM(cfg).eval()


def test_apply_teal_hook_mode(tmp_path):
    model = _tiny_model()
    ids = torch.randint(0, 100, (1, 6))
    with torch.no_grad():
        dense = model(ids).logits
    with pytest.raises(ValueError):
        patching.apply_teal(model)
    with pytest.raises(ValueError):
        patching.apply_teal(model, sparsity=0.4, thresholds={})
    thresholds = {0: {p: 0.01 for p in patching.PROJ_NAMES}, 1: {"q_proj": 0.2}}
    path = tmp_path / "thr.json"
    path.write_text(json.dumps({str(k): v for k, v in thresholds.items()}))
    sp = patching.apply_teal(model, thresholds_path=str(path))
    assert len(sp) == 14 and sp[(0, "down_proj")].threshold == 0.01
    assert sp[(1, "k_proj")].threshold == 0.0 and not sp[(1, "k_proj")].enabled
    seen = {}
    proj = model.model.layers[0].mlp.down_proj
    h = proj.register_forward_pre_hook(lambda m, a: seen.setdefault("x", a[0].clone()))
    with torch.no_grad():
        sparse = model(ids).logits
    h.remove()
    assert not torch.equal(dense, sparse)
    assert (seen["x"].abs() > 0).logical_and(seen["x"].abs() <= 0.01).sum() == 0   # hook ran first
    rep = patching.get_sparsity_report(model)
    assert 0.0 < rep[(0, "down_proj")] < 1.0 and rep[(1, "k_proj")] == 0.0
    patching.print_sparsity_report(model)
    patching.remove_teal(model)
    assert not hasattr(model, "_teal_sparsifiers")
    with torch.no_grad():
        assert torch.equal(model(ids).logits, dense)
    # uniform sparsity without calibration uses the reference's 0.1 * s rule
    sp = patching.apply_teal(model, sparsity=0.4)
    assert sp[(0, "q_proj")].threshold == pytest.approx(0.04)
    patching.remove_teal(model)


def test_prepare_weight_layout():
    from leankv_b200.teal.kernels.sparse_gemv import prepare_weight_for_sparse_gemv

    w = torch.randn(24, 10).half()
    wt = prepare_weight_for_sparse_gemv(w)
    assert wt.shape == w.shape and wt.stride() == (1, 24) and torch.equal(wt, w)


def test_paged_cache_page_accounting():
    from leankv_b200.turboquant.paged_cache import PagedKVCache

    c = PagedKVCache(num_layers=1, num_kv_heads=2, num_q_heads=8, max_pages=4, device="cpu")
    assert c.kv_data.shape == (1, 4, 2, 2, 800)
    assert [c._allocate_page() for _ in range(4)] == [3, 2, 1, 0]      # LIFO like the reference
    with pytest.raises(RuntimeError, match="out of pages"):
        c._allocate_page()
    assert c.get_pages_used() == 4
    c.reset()
    assert c.get_pages_used() == 0 and c.get_max_length() == 64
    with pytest.raises(RuntimeError):
        PagedKVCache(head_dim=64, device="cpu")


def test_threshold_files_round_trip_in_the_reference_format(tmp_path, capsys):
    """thresholds_s{NN}.json as the reference's calibration writes it (leankv/teal/greedy_opt.py:183-199):
    string layer keys, 0.0 = projection left dense; saved files load back and feed apply_teal."""
    from leankv_b200.teal.greedy_opt import load_thresholds, save_thresholds

    thr = {0: {p: 0.25 * (i + 1) for i, p in enumerate(patching.PROJ_NAMES)}, 1: {"q_proj": 0.0, "down_proj": 1.5}}
    path = tmp_path / "thresholds" / "thresholds_s40.json"
    save_thresholds(thr, str(path))
    assert "Saved thresholds" in capsys.readouterr().out
    on_disk = json.loads(path.read_text())
    assert set(on_disk) == {"0", "1"} and on_disk["1"] == {"q_proj": 0.0, "down_proj": 1.5}
    assert load_thresholds(str(path)) == thr
    # a file written by hand the way the reference does (keys already strings)
    ref_style = tmp_path / "ref.json"
    ref_style.write_text(json.dumps({"1": {"o_proj": 0.5}, "0": {"q_proj": 0.125}}, indent=2))
    assert load_thresholds(str(ref_style)) == {1: {"o_proj": 0.5}, 0: {"q_proj": 0.125}}
    model = _tiny_model()
    sp = patching.apply_teal(model, thresholds_path=str(path))
    assert sp[(0, "k_proj")].threshold == 0.5 and not sp[(1, "q_proj")].enabled
    assert sp[(1, "down_proj")].threshold == 1.5
    patching.remove_teal(model)


def test_argument_validation_of_the_decode_and_exchange_entry_points():
    """Glue kernels, batched glue kernels and the GEMV + all-reduce entry reject bad arguments with a
    status code before anything is launched (so this runs without a GPU)."""
    _no_device_for_made_up_pointers()
    lib = _native.lib()
    fake, odd = 0x10000, 0x10002
    assert lib.leankv_rmsnorm_f16(None, None, fake, fake, 4096, 1e-5, None) == -1
    assert lib.leankv_rmsnorm_f16(fake, None, fake, fake, 4100, 1e-5, None) == -2
    assert lib.leankv_rmsnorm_f16(fake, None, fake, fake, 1 << 20, 1e-5, None) == -6
    assert lib.leankv_rmsnorm_rows_f16(fake, None, fake, fake, 0, 4096, 1e-5, None) == -1
    assert lib.leankv_rmsnorm_rows_f16(odd, None, fake, fake, 4, 4096, 1e-5, None) == -2
    assert lib.leankv_rope_f16(fake, fake, fake, fake, fake, 32, 8, 64, None) == -5      # head_dim != 128
    assert lib.leankv_decode_begin(fake, fake, fake, 4100, 100, fake, None) == -2
    assert lib.leankv_decode_end(odd, 32768, fake, fake, 8, fake, None) == -2
    assert lib.leankv_decode_qkv_post(fake, fake, fake, fake, fake, fake, None, 4, fake, 32, 8, fake, None) == -1
    assert lib.leankv_batch_qkv_post(fake, 2, fake, fake, None, fake, fake, fake, fake, 4, fake, 32, 8, fake,
                                     None) == -1                                       # kv_indptr required
    assert lib.leankv_batch_decode_begin(fake, fake, fake, 4096, 100, 0, fake, fake, 4, fake, fake, fake,
                                         None) == -1
    assert lib.leankv_batch_decode_end(fake, 32770, 2, fake, fake, 8, fake, fake, None) == -2   # vocab % 8
    assert lib.leankv_silu_mul_f16(fake, fake, 2, 1001, None) == -2
    assert lib.leankv_xchg_advance(None, None) == -1
    assert lib.leankv_xchg_recv_bytes(4, 64, 4096) == 8 * 64 * 4 * 4096
    assert lib.leankv_xchg_recv_bytes(0, 64, 4096) == 0

    x = _native.Xchg()
    x.world, x.rank, x.n_slots, x.max_cols, x.max_wait_iters = 2, 0, 4, 4096, 100
    x.recv[0], x.recv[1] = fake, fake
    x.epoch, x.status = fake, fake
    ws = lib.leankv_sparse_gemv_workspace_bytes(4096, 2048)
    call = lambda xc, slot, n=4096: lib.leankv_sparse_gemv_allreduce_f16(
        fake, fake, fake, n, 2048, 0.1, None, fake, ws, None, ctypes.byref(xc), slot, None)
    assert call(x, 4) == -1                      # slot outside the area
    x.rank = 2
    assert call(x, 0) == -1                      # rank outside the world
    x.rank, x.world = 0, 9
    assert call(x, 0) == -1                      # more ranks than the struct can hold
    x.world, x.max_cols = 2, 1000
    assert call(x, 0) == -1                      # max_cols not a multiple of 256
    x.max_cols = 2048
    assert call(x, 0) == -1                      # N does not fit the receive area
    x.max_cols, x.recv[1] = 4096, None
    assert call(x, 0) == -1                      # a peer's area is missing
    x.recv[1], x.max_wait_iters = fake + 4, 100
    assert call(x, 0) == -1                      # receive area not 8-byte aligned
    assert lib.leankv_ipc_alloc(0, None, None) == -1 and lib.leankv_ipc_open(None, None) == -1
    assert lib.leankv_ipc_close(None) == -1 and lib.leankv_ipc_free(None) == -1


def test_argument_validation_of_the_prefill_attention_and_sharded_argmax_entry_points():
    """``leankv_tq_prefill_attn`` and ``leankv_decode_end_sharded`` reject bad arguments before any launch."""
    _no_device_for_made_up_pointers()
    lib = _native.lib()
    fake, odd = 0x10000, 0x10002
    need = lib.leankv_tq_prefill_attn_workspace_bytes(512, 0, 32, 8)
    assert need > lib.leankv_tq_decode_attn_workspace_bytes(512, 32, 8, 32)      # decode workspace + the page-table rows
    assert lib.leankv_tq_prefill_attn_workspace_bytes(0, 0, 32, 8) == 0
    assert lib.leankv_tq_prefill_attn_workspace_bytes(70000, 0, 32, 8) == 0      # more rows than one call takes
    assert lib.leankv_tq_prefill_attn_workspace_bytes(65535, (1 << 24) - 65535, 32, 8) == 0   # int32 page-table offsets
    call = lambda T=512, start=0, ws=fake, nbytes=need, q=fake: lib.leankv_tq_prefill_attn(
        q, fake, T, start, 32, 8, fake, 64, fake, fake, fake, fake, 0.088, ws, nbytes, None)
    assert call(T=-1) == -1
    assert call(start=-5) == -1
    assert call(T=0) == 0                          # nothing to do
    assert call(q=None) == -1
    assert call(T=70000) == -6
    assert call(ws=odd) == -2
    assert call(nbytes=need - 1) == -3

    x = _native.Xchg()
    x.world, x.rank, x.n_slots, x.max_cols, x.max_wait_iters = 2, 0, 4, 4096, 100
    x.recv[0], x.recv[1] = fake, fake
    x.epoch, x.status = fake, fake
    end = lambda xc, slot=3, vl=4096, logits=fake: lib.leankv_decode_end_sharded(
        logits, vl, 4096, fake, fake, 8, fake, ctypes.byref(xc), slot, None)
    assert end(x, slot=4) == -1                    # slot outside the area
    assert end(x, vl=4100) == -2                   # slice length not a multiple of 8
    assert end(x, logits=odd) == -2
    assert end(x, logits=None) == -1
    x.recv[1] = None
    assert end(x) == -1                            # a peer's area is missing
