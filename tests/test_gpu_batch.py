"""Batched decode: the batched glue kernels against their single-sequence forms on identical inputs
(bit for bit), and the whole batched step against single-sequence engines on the same weights."""

import ctypes

import pytest
import torch

from conftest import rel_l2
from leankv_b200 import _native
from leankv_b200.batch_engine import BatchDecodeEngine
from leankv_b200.engine import DecodeEngine, DecoderConfig

pytestmark = pytest.mark.gpu

CFG = DecoderConfig(vocab_size=1024, hidden_size=512, intermediate_size=1024, num_layers=2, num_q_heads=8,
                    num_kv_heads=2)


def _dev():
    return torch.device("cuda:0")


def _st():
    return torch.cuda.current_stream().cuda_stream


def test_rmsnorm_rows_equals_single_row_kernel():
    lib = _native.lib()
    g = torch.Generator(device=_dev()).manual_seed(0)
    rows, n = 5, 4096
    x = torch.randn(rows, n, device=_dev(), generator=g).half()
    d = torch.randn(rows, n, device=_dev(), generator=g).half()
    w = torch.randn(n, device=_dev(), generator=g).half()
    xa, ya = x.clone(), torch.empty_like(x)
    _native.check(lib.leankv_rmsnorm_rows_f16(xa.data_ptr(), d.data_ptr(), w.data_ptr(), ya.data_ptr(), rows, n,
                                              1e-5, _st()), "rows")
    for r in range(rows):
        xb, yb = x[r].clone(), torch.empty(n, dtype=torch.float16, device=_dev())
        _native.check(lib.leankv_rmsnorm_f16(xb.data_ptr(), d[r].data_ptr(), w.data_ptr(), yb.data_ptr(), n, 1e-5,
                                             _st()), "row")
        torch.cuda.synchronize()
        assert torch.equal(xa[r], xb) and torch.equal(ya[r], yb)


def test_silu_mul_rounding_points():
    lib = _native.lib()
    g = torch.Generator(device=_dev()).manual_seed(1)
    rows, inter = 7, 1024
    gu = (torch.randn(rows, 2 * inter, device=_dev(), generator=g) * 3).half()
    out = torch.empty(rows, inter, dtype=torch.float16, device=_dev())
    _native.check(lib.leankv_silu_mul_f16(gu.data_ptr(), out.data_ptr(), rows, inter, _st()), "silu_mul")
    torch.cuda.synchronize()
    gate, up = gu[:, :inter].float(), gu[:, inter:]
    want = (gate * torch.sigmoid(gate)).half() * up
    # __expf differs from torch's exp in the last bits: allow one fp16 ulp on the activation
    err = (out.float() - want.float()).abs()
    assert float((err / (want.float().abs() + 1e-3)).max()) < 3e-3
    assert rel_l2(out, want) < 1e-3


def test_batch_begin_builds_the_flat_page_table():
    lib = _native.lib()
    B, pps, hidden, vocab = 6, 9, 256, 50
    g = torch.Generator().manual_seed(2)
    table = torch.randn(vocab, hidden, generator=g).half().to(_dev())
    tokens = torch.tensor([3, 49, 0, 7, 7, 21], device=_dev())
    pos = torch.tensor([0, 15, 16, 47, 100, 143], dtype=torch.int32, device=_dev())
    bt = torch.randperm(B * pps, generator=g).to(torch.int32).reshape(B, pps).to(_dev())
    h = torch.zeros(B, hidden, dtype=torch.float16, device=_dev())
    indptr = torch.zeros(B + 1, dtype=torch.int32, device=_dev())
    flat = torch.full((B * pps,), -1, dtype=torch.int32, device=_dev())
    last = torch.zeros(B, dtype=torch.int32, device=_dev())
    _native.check(lib.leankv_batch_decode_begin(table.data_ptr(), tokens.data_ptr(), h.data_ptr(), hidden, vocab, B,
                                                pos.data_ptr(), bt.data_ptr(), pps, indptr.data_ptr(),
                                                flat.data_ptr(), last.data_ptr(), _st()), "begin")
    torch.cuda.synchronize()
    assert torch.equal(h, table[tokens])
    used = [int(p) // 16 + 1 for p in pos.tolist()]
    want_indptr = [0]
    for u in used:
        want_indptr.append(want_indptr[-1] + u)
    assert indptr.tolist() == want_indptr
    assert last.tolist() == [int(p) % 16 + 1 for p in pos.tolist()]
    want_flat = torch.cat([bt[b, :used[b]] for b in range(B)])
    assert torch.equal(flat[:want_indptr[-1]], want_flat)


def test_batch_decode_end_is_rowwise_argmax():
    lib = _native.lib()
    B, vocab, cap = 5, 4096, 12
    g = torch.Generator(device=_dev()).manual_seed(3)
    logits = torch.randn(B, vocab, device=_dev(), generator=g).half()
    logits[2, 100] = logits[2, 3000] = 9.0          # tie: lowest index wins
    tokens = torch.zeros(B, dtype=torch.int64, device=_dev())
    hist = torch.zeros(B, cap, dtype=torch.int64, device=_dev())
    pos = torch.arange(10, 10 + B, dtype=torch.int32, device=_dev())
    steps = torch.tensor([0, 1, 2, 3, 11], dtype=torch.int32, device=_dev())
    _native.check(lib.leankv_batch_decode_end(logits.data_ptr(), vocab, B, tokens.data_ptr(), hist.data_ptr(), cap,
                                              pos.data_ptr(), steps.data_ptr(), _st()), "end")
    torch.cuda.synchronize()
    want = logits.float().argmax(dim=-1)
    want[2] = 100
    assert torch.equal(tokens, want)
    assert pos.tolist() == list(range(11, 11 + B)) and steps.tolist() == [1, 2, 3, 4, 12]
    for b, s in enumerate([0, 1, 2, 3, 11]):
        assert int(hist[b, s]) == int(want[b])


def test_batch_qkv_post_is_bit_identical_to_single_sequence_kernel():
    """Same qkv rows, positions and pages through the batched launch and through one launch per sequence."""
    lib = _native.lib()
    B = 11
    eng = BatchDecodeEngine.random_init(CFG, _dev(), B, seed=1, max_seq_len=160)
    g = torch.Generator(device=_dev()).manual_seed(4)
    qkv = torch.randn(B, eng.n_qkv, device=_dev(), generator=g).half()
    pos = torch.tensor([0, 1, 15, 16, 17, 31, 32, 77, 100, 158, 159], dtype=torch.int32, device=_dev())
    eng.pos.copy_(pos)
    # page table of this step
    _native.check(lib.leankv_batch_decode_begin(eng.w["embed"].data_ptr(), eng.tokens.data_ptr(), eng.h.data_ptr(),
                                                CFG.hidden_size, CFG.vocab_size, B, eng.pos.data_ptr(),
                                                eng.block_table.data_ptr(), eng.pps, eng.kv_indptr.data_ptr(),
                                                eng.kv_page_indices.data_ptr(), eng.kv_last.data_ptr(), _st()), "begin")
    base = torch.randint(0, 256, eng.pools[0].shape, dtype=torch.uint8, device=_dev(), generator=g)
    pool_a, pool_b = base.clone(), base.clone()
    q_a = torch.zeros(B, eng.nq, 128, dtype=torch.float32, device=_dev())
    q_b = torch.zeros_like(q_a)
    _native.check(lib.leankv_batch_qkv_post(qkv.data_ptr(), B, eng.inv_freq.data_ptr(), eng.pos.data_ptr(),
                                            eng.kv_indptr.data_ptr(), eng.Pi_k_t[0].data_ptr(),
                                            eng.Pi_v_t[0].data_ptr(), eng.bounds.data_ptr(), pool_a.data_ptr(),
                                            eng.max_pages, eng.kv_page_indices.data_ptr(), eng.nq, eng.nkv,
                                            q_a.data_ptr(), _st()), "batch post")
    state = torch.zeros(8, dtype=torch.int32, device=_dev())
    for b in range(B):
        state[0] = pos[b]
        pages = eng.block_table[b].contiguous()
        _native.check(lib.leankv_decode_qkv_post(qkv[b].data_ptr(), eng.inv_freq.data_ptr(), state.data_ptr(),
                                                 eng.Pi_k_t[0].data_ptr(), eng.Pi_v_t[0].data_ptr(),
                                                 eng.bounds.data_ptr(), pool_b.data_ptr(), eng.max_pages,
                                                 pages.data_ptr(), eng.nq, eng.nkv, q_b[b].data_ptr(), _st()), "post")
        torch.cuda.synchronize()
    assert torch.equal(q_a, q_b)
    assert torch.equal(pool_a, pool_b)
    assert not torch.equal(pool_a, base)


def test_batched_step_matches_single_sequence_engines():
    """Dense projections either way (no thresholds): library GEMM rows vs the GEMV kernel differ in
    summation order only, so logits agree to fp16 rounding while tokens are teacher-forced."""
    B, T, n_new = 3, 40, 6
    g = torch.Generator().manual_seed(5)
    prompts = torch.randint(0, CFG.vocab_size, (B, T), generator=g)
    forced = torch.randint(0, CFG.vocab_size, (n_new, B), generator=g)

    eng = BatchDecodeEngine.random_init(CFG, _dev(), B, seed=9, max_seq_len=96)
    eng.prefill(prompts)
    got = [eng.prefill_logits.float().cpu()]
    for i in range(n_new):
        eng.tokens.copy_(forced[i].to(_dev()))
        eng.step()
        torch.cuda.synchronize()
        got.append(eng.logits.float().cpu())
    assert eng.pos.tolist() == [T + n_new] * B
    # 1 begin + 1 norm + per block (post, attention, norm, silu_mul, norm) + argmax; 4 GEMMs per block + lm_head
    assert eng.launches_per_step == 2 + 5 * CFG.num_layers + 1
    assert eng.gemms_per_step == 4 * CFG.num_layers + 1

    for b in range(B):
        one = DecodeEngine.random_init(CFG, _dev(), seed=9, max_seq_len=96)
        one.prefill(prompts[b].tolist())
        assert rel_l2(got[0][b], one.prefill_logits.float().cpu()) < 5e-3
        for i in range(n_new):
            one.token.fill_(int(forced[i, b]))
            one.step()
            torch.cuda.synchronize()
            err = rel_l2(got[i + 1][b], one.logits.float().cpu())
            assert err < 2e-2, (b, i, err)


def test_generate_returns_history_and_graph_equals_eager():
    B, T = 4, 33
    g = torch.Generator().manual_seed(6)
    prompts = torch.randint(0, CFG.vocab_size, (B, T), generator=g)
    a = BatchDecodeEngine.random_init(CFG, _dev(), B, seed=2, max_seq_len=64)
    toks = a.generate(prompts, 8)
    assert toks.shape == (B, 8)
    b = BatchDecodeEngine.random_init(CFG, _dev(), B, seed=2, max_seq_len=64)
    b.prefill(prompts)
    for _ in range(7):
        b.step(use_graph=False)
    torch.cuda.synchronize()
    assert torch.equal(toks, b.history[:, :8])
    assert a.kv_bytes_per_sequence(4096) == 256 * 2 * CFG.num_layers * CFG.num_kv_heads * 800
