"""TEAL sparse GEMV / SwiGLU kernels (through the C ABI) against the oracle and the reference goldens."""

import ctypes

import numpy as np
import pytest
import torch

from conftest import rel_l2
from leankv_b200 import _native, workloads
from leankv_b200.teal.kernels.sparse_gemv import (batched_sparse_gemm, prepare_weight_for_sparse_gemv,
                                                  sparse_gemv, sparse_swiglu)
from oracle import teal as oteal

pytestmark = pytest.mark.gpu
TOL = 1e-3   # rel-L2 bound for fp16 GEMV outputs


def _dev():
    return torch.device("cuda:0")


def _raw_gemv(wt, x, t, bias=None, residual=None, segs=None):
    """Direct C-ABI call; returns (y, active_elems)."""
    lib = _native.lib()
    z, n = wt.shape
    y = torch.empty(n, dtype=torch.float16, device=wt.device)
    ws = torch.zeros(max(lib.leankv_sparse_gemv_workspace_bytes(n, z), 256), dtype=torch.uint8, device=wt.device)
    cnt = torch.zeros(1, dtype=torch.int64, device=wt.device)
    st = torch.cuda.current_stream().cuda_stream
    if segs is None:
        rc = lib.leankv_sparse_gemv_f16(wt.data_ptr(), x.data_ptr(), y.data_ptr(), n, z, float(t),
                                        _native.ptr(bias), _native.ptr(residual), ws.data_ptr(), ws.numel(),
                                        cnt.data_ptr(), st)
    else:
        rc = lib.leankv_sparse_gemv_seg_f16(wt.data_ptr(), x.data_ptr(), y.data_ptr(), n, z,
                                            ctypes.byref(segs), _native.ptr(bias), _native.ptr(residual),
                                            ws.data_ptr(), ws.numel(), cnt.data_ptr(), st)
    _native.check(rc, "sparse gemv")
    torch.cuda.synchronize()
    assert int(ws[:4 * ((n + 255) // 256)].sum()) == 0, "arrival counters must be left zeroed"
    return y, int(cnt.item())


def test_small_and_ragged_cases_vs_reference(golden_teal):
    for i, (n, z, s, seed) in enumerate(golden_teal["small_cases"]):
        n, z = int(n), int(z)
        c = workloads.sparse_gemv_case(n, z, float(s), int(seed), device=_dev())
        t = float(golden_teal[f"small{i}_threshold"])
        assert c.threshold == t
        wt = c.weight.t().contiguous()
        y, active = _raw_gemv(wt, c.x.reshape(-1).contiguous(), t)
        mask = golden_teal[f"small{i}_mask"]
        n_act = int(mask.sum()) if t > 0 else int((c.x != 0).sum())   # t == 0 still skips exact zeros
        assert active == n_act * n, f"case {i}: mask differs from the reference's"
        want32 = torch.from_numpy(golden_teal[f"small{i}_y_fp32"]).reshape(-1)
        if n_act == 0:
            assert torch.count_nonzero(y) == 0
            continue
        assert rel_l2(y.cpu(), want32) < TOL, f"case {i}"
        # fp16 rounding of an fp32-accumulated sum: at most one fp16 ulp from the fp32 reference
        ulp = torch.from_numpy(np.spacing(np.abs(want32.numpy()).astype(np.float16)).astype(np.float32))
        # (+1e-5: where terms cancel, the two fp32 summation orders differ by more than the tiny result's ulp)
        assert torch.all((y.cpu().float() - want32).abs() <= ulp + 1e-5)
        # the API wrapper gives the same bits
        y2 = sparse_gemv(c.x.reshape(1, 1, z), prepare_weight_for_sparse_gemv(c.weight), t)
        assert y2.shape == (1, 1, n) and torch.equal(y2.reshape(-1), y)


def test_config1_full_size(golden_teal):
    c = workloads.sparse_gemv_case(device=_dev())
    wt = c.weight.t().contiguous()
    y, active = _raw_gemv(wt, c.x.reshape(-1).contiguous(), c.threshold)
    assert active == int(golden_teal["c1_n_active"]) * 4096
    assert rel_l2(y.cpu(), golden_teal["c1_y_fp32"]) < TOL
    assert rel_l2(y.cpu(), golden_teal["c1_y_fp16"]) < TOL
    y_again, _ = _raw_gemv(wt, c.x.reshape(-1).contiguous(), c.threshold)
    assert torch.equal(y, y_again), "fixed-order split-K must be bit-reproducible"
    # mask monotonicity in the threshold
    counts = [_raw_gemv(wt, c.x.reshape(-1).contiguous(), t)[1] for t in (0.1, 0.5, 1.0, 3.0, 1e9)]
    assert counts == sorted(counts, reverse=True) and counts[-1] == 0
    # linearity in x over a fixed mask: doubling x (and t) doubles y exactly in fp16
    y2, _ = _raw_gemv(wt, (c.x.reshape(-1) * 2).contiguous(), c.threshold * 2)
    assert torch.equal(y2, y * 2)


def test_config2_fused_swiglu_full_size(golden_teal):
    c = workloads.swiglu_case(device=_dev())
    wg, wu = prepare_weight_for_sparse_gemv(c.w_gate), prepare_weight_for_sparse_gemv(c.w_up)
    y = sparse_swiglu(c.x.reshape(1, 1, -1), wg, wu, c.threshold, c.threshold).reshape(-1)
    assert rel_l2(y.cpu(), golden_teal["c2_y_fp32"].reshape(-1)) < TOL
    assert rel_l2(y.cpu(), golden_teal["c2_y_fp16"].reshape(-1)) < TOL
    # equals two sparse GEMVs + act_fn(gate) * up, the way the reference composes it
    g = sparse_gemv(c.x.reshape(1, 1, -1), wg, c.threshold)
    u = sparse_gemv(c.x.reshape(1, 1, -1), wu, c.threshold)
    # (the fused kernel splits the input channels differently, so its fp32 sums round differently)
    composed = (torch.nn.functional.silu(g) * u).reshape(-1)
    assert rel_l2(y.cpu(), composed.cpu()) < TOL and (y != composed).float().mean() < 0.05
    assert torch.equal(y, sparse_swiglu(c.x.reshape(1, 1, -1), wg, wu, c.threshold, c.threshold).reshape(-1))


def test_swiglu_distinct_thresholds_and_ragged():
    for (n, z, tg, tu, seed) in ((264, 100, 0.2, 0.9, 1), (512, 37, 1.5, 0.1, 2), (8, 3, 0.0, 0.0, 3)):
        c = workloads.swiglu_case(n, z, 0.4, seed, device=_dev())
        wg, wu = prepare_weight_for_sparse_gemv(c.w_gate), prepare_weight_for_sparse_gemv(c.w_up)
        y = sparse_swiglu(c.x.reshape(1, 1, -1), wg, wu, tg, tu).reshape(-1)
        want = oteal.swiglu(c.x.cpu(), c.w_gate.cpu(), c.w_up.cpu(), tg, tu, accumulate="fp32").reshape(-1)
        assert rel_l2(y.cpu(), want) < 2 * TOL   # three fp16 roundings on the reference path


def test_threshold_is_strict_and_rounded_to_fp16():
    dev = _dev()
    z, n = 64, 256
    w = torch.ones(n, z, dtype=torch.float16, device=dev)
    wt = w.t().contiguous()
    x = torch.zeros(z, dtype=torch.float16, device=dev)
    edge = 1.0 + 2.0 ** -10
    x[3], x[10], x[20] = edge, -edge, 1.0 + 2.0 ** -9
    # |x| == t is dropped (strict >)
    y, active = _raw_gemv(wt, x, edge)
    assert active == 1 * n and float(y[0]) == pytest.approx(1.0 + 2.0 ** -9, abs=1e-3)
    # a threshold just below the fp16 value rounds up to it: torch compares in fp16, so do we
    y, active = _raw_gemv(wt, x, edge - 1e-5)
    assert active == 1 * n
    ref = oteal.sparsify(x.cpu(), edge - 1e-5)
    assert int((ref != 0).sum()) == 1
    # negative threshold keeps everything non-NaN, including zeros
    y, active = _raw_gemv(wt, x, -1.0)
    assert active == z * n


def test_segments_bias_residual():
    dev = _dev()
    gen = torch.Generator(device="cpu").manual_seed(4)
    z, n = 300, 1024 + 256 + 512
    w = (torch.randn(n, z, generator=gen) * 0.05).half().to(dev)
    x = torch.randn(z, generator=gen).half().to(dev)
    bias = torch.randn(n, generator=gen).half().to(dev)
    res = torch.randn(n, generator=gen).half().to(dev)
    wt = w.t().contiguous()
    segs = _native.Segments()
    segs.n_segments = 3
    ends, thr = (1024, 1280, n), (0.2, 0.8, 1.4)
    for i in range(3):
        segs.seg_end[i], segs.threshold[i] = ends[i], thr[i]
    y, active = _raw_gemv(wt, x, 0.0, segs=segs)
    start, want_active = 0, 0
    for e, t in zip(ends, thr):
        part, a = _raw_gemv(wt[:, start:e].contiguous(), x, t)
        assert torch.equal(y[start:e], part)
        want_active += a
        start = e
    assert active == want_active
    yb, _ = _raw_gemv(wt, x, 0.5, bias=bias, residual=res)
    y0, _ = _raw_gemv(wt, x, 0.5)
    assert torch.equal(yb, res + (y0 + bias))


def test_batched_wrapper_and_dtype():
    dev = _dev()
    c = workloads.sparse_gemv_case(520, 264, 0.5, 8, device=dev)
    w = prepare_weight_for_sparse_gemv(c.weight)
    xb = torch.stack([c.x.reshape(-1), c.x.reshape(-1) * 0.5, -c.x.reshape(-1)])
    yb = batched_sparse_gemm(xb, w, c.threshold)
    assert yb.shape == (3, 520)
    for i in range(3):
        want = oteal.sparse_linear(xb[i].cpu().reshape(1, -1), c.weight.cpu(), c.threshold, "fp32")
        assert rel_l2(yb[i].cpu(), want.reshape(-1)) < TOL
    y32 = sparse_gemv(c.x.float().reshape(1, 1, -1), w, c.threshold)
    assert y32.dtype == torch.float32
    with pytest.raises(ValueError, match="column-major"):
        sparse_gemv(c.x.reshape(1, 1, -1), c.weight, c.threshold)


def test_apply_teal_kernel_mode_matches_hook_mode():
    from transformers import MistralConfig, MistralForCausalLM

    from leankv_b200.teal import patching

    dev = _dev()
    torch.manual_seed(0)
    cfg = MistralConfig(vocab_size=512, hidden_size=256, intermediate_size=768, num_hidden_layers=2,
                        num_attention_heads=4, num_key_value_heads=2, head_dim=64,
                        max_position_embeddings=128)
    thresholds = {l: {p: 0.25 if p != "down_proj" else 0.02 for p in patching.PROJ_NAMES} for l in range(2)}
    ids = torch.randint(0, 512, (1, 9), device=dev)
    logits = {}
    for mode in ("hook", "kernel", "fused"):
        torch.manual_seed(0)
        model = MistralForCausalLM(cfg).half().to(dev).eval()
        with torch.no_grad():
            # dense prefill in every mode: the kernel mode of the reference is dense whenever more
            # than one token is in flight (patching.py:178-180), the hook mode is not
            out = model(ids[:, :8], use_cache=True)
            patching.apply_teal(model, thresholds=thresholds, use_triton=(mode != "hook"),
                                fuse_mlp=(mode == "fused"))
            step = model(ids[:, 8:], past_key_values=out.past_key_values, use_cache=True)
        logits[mode] = step.logits.float().cpu()
        if mode != "hook":
            assert model.model.layers[0].mlp.down_proj._teal_patched
    assert rel_l2(logits["kernel"], logits["hook"]) < 5e-3
    assert rel_l2(logits["fused"], logits["kernel"]) < 5e-3


def _allreduce_gemv(wt, x, t, residual, xchg_c, slot):
    lib = _native.lib()
    z, n = wt.shape
    y = torch.empty(n, dtype=torch.float16, device=wt.device)
    ws = torch.zeros(max(lib.leankv_sparse_gemv_workspace_bytes(n, z), 256), dtype=torch.uint8, device=wt.device)
    rc = lib.leankv_sparse_gemv_allreduce_f16(wt.data_ptr(), x.data_ptr(), y.data_ptr(), n, z, float(t),
                                              _native.ptr(residual), ws.data_ptr(), ws.numel(), None,
                                              ctypes.byref(xchg_c), slot, torch.cuda.current_stream().cuda_stream)
    _native.check(rc, "gemv + all-reduce")
    torch.cuda.synchronize()
    return y


def test_allreduce_gemv_with_one_rank_equals_plain_gemv():
    """A single rank exchanges with itself: same publish / flag / wait / ordered-sum code path, and the
    sum of one partial is that partial, so the output must equal the plain kernel's bit for bit."""
    from leankv_b200.peer_exchange import PeerExchange

    dev = _dev()
    gen = torch.Generator(device="cpu").manual_seed(11)
    ex = PeerExchange(dev, n_slots=3, max_cols=4096)
    try:
        for step, (z, n, t) in enumerate([(14336, 4096, 0.6), (300, 1000, 0.2), (4096, 4096, -1.0)]):
            w = (torch.randn(n, z, generator=gen) * 0.02).half().to(dev)
            x = torch.randn(z, generator=gen).half().to(dev)
            res = torch.randn(n, generator=gen).half().to(dev)
            wt = w.t().contiguous()
            want, _ = _raw_gemv(wt, x, t, residual=res)
            for slot in range(3):
                got = _allreduce_gemv(wt, x, t, res, ex.c, slot)
                assert torch.equal(got, want), (step, slot)
            ex.advance(torch.cuda.current_stream().cuda_stream)     # next step: flags of this one are stale
        assert not ex.timed_out()
        lib = _native.lib()
        bad = _native.Xchg.from_buffer_copy(ex.c)
        bad.rank = 1
        y = torch.empty(256, dtype=torch.float16, device=dev)
        ws = torch.zeros(lib.leankv_sparse_gemv_workspace_bytes(256, 64) + 256, dtype=torch.uint8, device=dev)
        assert lib.leankv_sparse_gemv_allreduce_f16(wt.data_ptr(), x.data_ptr(), y.data_ptr(), 256, 64, 0.0, None,
                                                    ws.data_ptr(), ws.numel(), None, ctypes.byref(bad), 0,
                                                    None) == -1          # rank outside the world
        assert lib.leankv_sparse_gemv_allreduce_f16(wt.data_ptr(), x.data_ptr(), y.data_ptr(), 256, 64, 0.0, None,
                                                    ws.data_ptr(), ws.numel(), None, ctypes.byref(ex.c), 3,
                                                    None) == -1          # slot outside the area
    finally:
        ex.close()


def test_allreduce_wait_gives_up_when_a_peer_never_arrives():
    """Two-rank exchange where nobody plays rank 1 (its area is a second local buffer): the bounded
    wait runs out, the kernel returns, the status word is set and later launches skip their waits."""
    lib = _native.lib()
    dev = _dev()
    world, slots, cols = 2, 2, 1024
    recv = [torch.zeros(lib.leankv_xchg_recv_bytes(world, slots, cols), dtype=torch.uint8, device=dev)
            for _ in range(world)]
    epoch = torch.ones(1, dtype=torch.int32, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    xc = _native.Xchg()
    xc.world, xc.rank, xc.n_slots, xc.max_cols, xc.max_wait_iters = world, 0, slots, cols, 2000
    for r in range(world):
        xc.recv[r] = recv[r].data_ptr()
    xc.epoch, xc.status = epoch.data_ptr(), status.data_ptr()
    gen = torch.Generator(device="cpu").manual_seed(12)
    wt = (torch.randn(512, 1024, generator=gen) * 0.02).half().to(dev)
    x = torch.randn(512, generator=gen).half().to(dev)
    y = _allreduce_gemv(wt, x, 0.1, None, xc, 0)
    assert int(status.item()) == 1
    assert bool(torch.isfinite(y.float()).all())
    # rank 0's values reached the absent peer's area, tagged with the epoch, though nothing came back
    plain, _ = _raw_gemv(wt, x, 0.1)
    words = recv[1].view(torch.int32).reshape(-1, 2)[:1024]
    assert rel_l2(words[:, 0].contiguous().view(torch.float32), plain) < 1e-3
    assert bool((words[:, 1] == 1).all())
    y2 = _allreduce_gemv(wt, x, 0.1, None, xc, 1)          # sticky status: returns without polling
    assert int(status.item()) == 1 and bool(torch.isfinite(y2.float()).all())
    torch.cuda.synchronize()


def test_one_workspace_serves_projections_of_different_widths():
    """A decode step runs all its projections through one workspace. The widest (the output head: 128
    column slices at vocabulary 32768, 501 at 128256) must still find its arrival counters at zero after
    narrower projections have left their partial sums in the same buffer."""
    lib = _native.lib()
    dev = torch.device("cuda:0")
    gen = torch.Generator(device=dev).manual_seed(11)
    shapes = [(6144, 512), (14336, 512), (512, 14336), (32768, 512), (128256, 512)]     # (N, Z)
    need = max(lib.leankv_sparse_gemv_workspace_bytes(n, z) for n, z in shapes)
    need = max(need, lib.leankv_sparse_swiglu_workspace_bytes(14336, 512))
    ws = torch.zeros(need, dtype=torch.uint8, device=dev)
    st = torch.cuda.current_stream().cuda_stream
    mats = {(n, z): (torch.randn(z, n, device=dev, generator=gen) * 0.05).half() for n, z in shapes}
    xs = {z: torch.randn(z, device=dev, generator=gen).half() for z in {z for _, z in shapes}}
    for _ in range(2):                                           # second round: everything has been used before
        for n, z in shapes:
            y = torch.full((n,), float("nan"), dtype=torch.float16, device=dev)
            _native.check(lib.leankv_sparse_gemv_f16(mats[(n, z)].data_ptr(), xs[z].data_ptr(), y.data_ptr(), n, z,
                                                     0.25, None, None, ws.data_ptr(), ws.numel(), None, st), "gemv")
            xm = xs[z].float() * (xs[z].abs().float() > 0.25)
            want = xm @ mats[(n, z)].float()
            assert torch.isfinite(y).all(), (n, z)
            assert rel_l2(y.cpu(), want.cpu()) < 1e-3, (n, z)
        g = torch.full((14336,), float("nan"), dtype=torch.float16, device=dev)
        _native.check(lib.leankv_sparse_swiglu_f16(mats[(14336, 512)].data_ptr(), mats[(14336, 512)].data_ptr(),
                                                   xs[512].data_ptr(), g.data_ptr(), 14336, 512, 0.25, 0.25,
                                                   ws.data_ptr(), ws.numel(), None, st), "swiglu")
        assert torch.isfinite(g).all()


_PREFETCH_SNIPPET = r"""
import hashlib, sys, torch
sys.path.insert(0, %(root)r)
from leankv_b200 import workloads
from leankv_b200.teal.kernels.sparse_gemv import prepare_weight_for_sparse_gemv, sparse_gemv, sparse_swiglu
dev = torch.device("cuda:0")
c = workloads.sparse_gemv_case(device=dev)
y1 = sparse_gemv(c.x.reshape(1, 1, -1), prepare_weight_for_sparse_gemv(c.weight), c.threshold)
s = workloads.swiglu_case(device=dev)
y2 = sparse_swiglu(s.x.reshape(1, 1, -1), prepare_weight_for_sparse_gemv(s.w_gate), prepare_weight_for_sparse_gemv(s.w_up),
                   s.threshold, s.threshold)
torch.cuda.synchronize()
print("OUT", hashlib.sha256(y1.cpu().numpy().tobytes() + y2.cpu().numpy().tobytes()).hexdigest())
"""


def test_weight_prefetch_budget_never_changes_a_result():
    """The kernels ask some of their weight rows into L2 ahead of the previous kernel's completion
    (LEANKV_GEMV_PREFETCH_KB, read once per process): a hint, so configs 1 and 2 must come out bit for bit the
    same with the prefetch off, at its default and with every row of a CTA's range asked for."""
    import os
    import subprocess
    import sys

    from conftest import ROOT

    out = {}
    for name, env in (("off", {"LEANKV_GEMV_PREFETCH_KB": "0"}), ("default", {}),
                      ("all", {"LEANKV_GEMV_PREFETCH_KB": "512", "LEANKV_GEMV_PREFETCH_PCT": "100"})):
        full = {k: v for k, v in os.environ.items() if not k.startswith("LEANKV_GEMV_PREFETCH")}
        full.update(env)
        r = subprocess.run([sys.executable, "-c", _PREFETCH_SNIPPET % {"root": ROOT}], env=full, capture_output=True,
                           text=True, timeout=600)
        assert r.returncode == 0, r.stderr[-2000:]
        out[name] = [ln for ln in r.stdout.splitlines() if ln.startswith("OUT")][-1].split()[1]
    assert out["off"] == out["default"] == out["all"]
