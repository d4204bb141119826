"""The CUDA-graph decode loop against HuggingFace + the oracle's TEAL hooks and TurboQuant cache on the same weights."""

import pytest
import torch

from conftest import rel_l2
from leankv_b200.engine import DecodeEngine, DecoderConfig, PROJ_NAMES
from leankv_b200.turboquant.cache import TurboQuantCache
from oracle import teal as oteal, turboquant as otq

pytestmark = pytest.mark.gpu


def _dev():
    return torch.device("cuda:0")


def _hf_model(layers=2, scale=1.0):
    from transformers import MistralConfig, MistralForCausalLM

    torch.manual_seed(0)
    cfg = MistralConfig(vocab_size=512, hidden_size=512, intermediate_size=1024, num_hidden_layers=layers,
                        num_attention_heads=8, num_key_value_heads=2, head_dim=128,
                        max_position_embeddings=256, rope_theta=1e6, rms_norm_eps=1e-5,
                        tie_word_embeddings=False)
    model = MistralForCausalLM(cfg)
    for p in model.parameters():            # scale > 1: sharper attention, logits far from uniform
        if p.dim() == 2:
            p.data.mul_(scale)
    return model.half().to(_dev()).eval()


class OracleCache(TurboQuantCache):
    """Quantize-on-append cache built from the oracle's torch restatement (fp16 norms, like the pool)."""

    def __init__(self, num_layers, device):
        super().__init__(bits=3, head_dim=128, num_layers=num_layers, hot_buffer_size=0, device=device)
        self.store = [None] * num_layers
        self.raw = [[] for _ in range(num_layers)]     # (k, v) exactly as the model handed them over

    def update(self, key_states, value_states, layer_idx, cache_kwargs=None):
        if layer_idx == 0:
            self._seen_tokens += key_states.shape[2]
        self._seq_lengths[layer_idx] += key_states.shape[2]
        self.raw[layer_idx].append((key_states.clone(), value_states.clone()))
        outs = []
        for which, x, quant in ((0, key_states, self.key_quantizers[layer_idx]),
                                (1, value_states, self.val_quantizers[layer_idx])):
            packed, norms, _, _ = otq.quantize(x.float(), quant.Pi, quant.decision_boundaries, 3)
            deq = otq.dequantize(packed, norms.half().float(), quant.Pi, quant.centroids, 3, 128).half()
            prev = self.store[layer_idx][which] if self.store[layer_idx] is not None else None
            outs.append(deq if prev is None else torch.cat([prev, deq], dim=2))
        self.store[layer_idx] = outs
        return outs[0], outs[1]


def _reference_run(model, prompt, n_new, thresholds):
    """HF forward with the oracle cache; oracle TEAL hooks are active on decode steps only
    (the reference's kernel mode is dense at prefill, patching.py:178-180)."""
    cache = OracleCache(model.config.num_hidden_layers, _dev())
    ids = torch.tensor([prompt], device=_dev())
    logits, tokens = [], []
    with torch.no_grad():
        out = model(ids, past_key_values=cache, use_cache=True)
        logits.append(out.logits[0, -1].float().cpu())
        tokens.append(int(out.logits[0, -1].float().argmax()))
        hooks = []
        if thresholds is not None:
            for l, layer in enumerate(model.model.layers):
                for p in PROJ_NAMES:
                    mod = getattr(layer.self_attn if p in ("q_proj", "k_proj", "v_proj", "o_proj") else layer.mlp, p)
                    t = thresholds[l][p]
                    hooks.append(mod.register_forward_pre_hook(
                        lambda m, a, t=t: (oteal.sparsify(a[0], t),) + a[1:]))
        for _ in range(n_new - 1):
            out = model(torch.tensor([[tokens[-1]]], device=_dev()), past_key_values=cache, use_cache=True)
            logits.append(out.logits[0, -1].float().cpu())
            tokens.append(int(out.logits[0, -1].float().argmax()))
        for h in hooks:
            h.remove()
    return tokens, logits


def _engine_run(engine, prompt, n_new, follow_tokens=None, use_graph=True):
    """Step the engine; when ``follow_tokens`` is given, feed those tokens (teacher forcing) so that
    logits stay comparable even if an argmax near-tie picks another token."""
    logits, tokens = [], []
    tokens.append(engine.prefill(prompt))
    logits.append(engine.prefill_logits.float().cpu())
    for i in range(n_new - 1):
        if follow_tokens is not None:
            engine.token.fill_(follow_tokens[i])
        engine.step(use_graph=use_graph)
        torch.cuda.synchronize()
        logits.append(engine.logits.float().cpu())
        tokens.append(int(engine.token.item()))
    return tokens, logits


@pytest.mark.parametrize("sparse", [False, True])
def test_engine_matches_hf_with_oracle_hooks_and_cache(sparse):
    """End to end against HF + oracle hooks + oracle cache. The two paths compute k/v with different
    GEMM kernels; a last-bit difference in k flips a 3-bit code now and then, so agreement is
    statistical (a few 1e-3 at this model scale), not bitwise."""
    model = _hf_model()
    gen = torch.Generator().manual_seed(1)
    prompt = torch.randint(0, 512, (37,), generator=gen).tolist()
    engine = DecodeEngine.from_hf(model, max_seq_len=128)
    thresholds = engine.calibrate_thresholds(prompt, 0.4) if sparse else None
    if sparse:
        assert set(thresholds[0]) == set(PROJ_NAMES) and all(v > 0 for v in thresholds[1].values())
    n_new = 24
    ref_tokens, ref_logits = _reference_run(model, prompt, n_new, thresholds)
    eng_tokens, eng_logits = _engine_run(engine, prompt, n_new, follow_tokens=ref_tokens)
    errs = [rel_l2(e, r) for e, r in zip(eng_logits, ref_logits)]
    print("per-step logits rel-L2:", [f"{e:.1e}" for e in errs])
    # A magnitude threshold is a discontinuity: a last-bit difference in an activation next to the
    # threshold switches a whole weight column on or off, so with TEAL the two paths drift apart much
    # faster than without (the identical-input check below is the strict one for the sparse path).
    bound = (0.3, 0.2) if sparse else (3e-2, 1.5e-2)
    assert max(errs) < bound[0] and sum(errs) / len(errs) < bound[1]
    if sparse:
        # the counter says ~60 % of the projection weights were streamed on the decode steps
        streamed = engine.bytes_streamed()
        cfg = engine.cfg
        per_layer = 2 * (cfg.hidden_size * engine.n_qkv + engine.nq * 128 * cfg.hidden_size
                         + 3 * cfg.hidden_size * cfg.intermediate_size)
        dense = (n_new - 1) * (cfg.num_layers * per_layer + 2 * cfg.hidden_size * cfg.vocab_size)
        assert 0.45 < streamed / dense < 0.85


def test_decode_step_matches_dense_prompt_pass_on_a_peaked_model():
    """Kernel decode step (GEMV, rope, append, paged attention, norms) against the library-GEMM
    prompt pass of the same engine over the same tokens, on a model with sharp attention
    (weights x3). Only the newest token's k/v come from different GEMM kernels."""
    model = _hf_model(scale=3.0)
    gen = torch.Generator().manual_seed(2)
    ids = torch.randint(0, 512, (60,), generator=gen).tolist()
    engine = DecodeEngine.from_hf(model, max_seq_len=128)
    errs = []
    for T in (17, 32, 33, 59):
        engine.prefill(ids[:T])
        engine.token.fill_(ids[T])
        engine.step()
        torch.cuda.synchronize()
        got = engine.logits.float().cpu()
        with torch.no_grad():
            x = engine._dense_forward(torch.tensor(ids[:T + 1], device=_dev()), write_cache=False)
            want = (x @ engine.w["lm_head_t"]).float().cpu()
        errs.append(rel_l2(got, want))
        # and against the same step recomputed with library ops over the pool as the step left it
        # (same codes on both sides: rounding differences only, hence the tighter bound)
        assert rel_l2(got, engine.dense_step_reference(ids[T], T).cpu()) < 5e-3, T
    print("decode step vs dense pass rel-L2:", [f"{e:.1e}" for e in errs])
    assert max(errs) < 3e-2


def test_graph_replay_equals_eager_and_generate():
    model = _hf_model()
    prompt = list(range(3, 50))
    a = DecodeEngine.from_hf(model, max_seq_len=128)
    th = a.calibrate_thresholds(prompt, 0.4)
    b = DecodeEngine.from_hf(model, max_seq_len=128, thresholds=th)
    ta, la = _engine_run(a, prompt, 20, use_graph=True)
    tb, lb = _engine_run(b, prompt, 20, use_graph=False)
    assert ta == tb
    assert all(torch.equal(x, y) for x, y in zip(la, lb))
    assert a.generate(prompt, 20, stream_to_host=True) == ta
    assert a.generate(prompt, 20, stream_to_host=False) == ta
    assert a.launches_per_step == 1 + 6 * a.cfg.num_layers + 2
    # the pool holds prompt + generated tokens at 50 bytes per vector
    assert a.kv_bytes_per_token() == 2 * 2 * 2 * 50
    with pytest.raises(ValueError):
        a.prefill(list(range(128)))


def test_random_init_engine_runs_and_is_dense_without_thresholds():
    cfg = DecoderConfig(vocab_size=1024, hidden_size=512, intermediate_size=1024, num_layers=2,
                        num_q_heads=8, num_kv_heads=2)
    eng = DecodeEngine.random_init(cfg, _dev(), seed=3, max_seq_len=96)
    toks = eng.generate(list(range(40)), 16)
    assert len(toks) == 16 and all(0 <= t < 1024 for t in toks)
    eng.active_elems.zero_()
    eng.step()
    torch.cuda.synchronize()
    per_layer = 512 * eng.n_qkv + eng.nq * 128 * 512 + 3 * 512 * 1024
    assert eng.bytes_streamed() == 2 * (2 * per_layer + 512 * 1024)


def test_each_stage_matches_hf_on_identical_inputs():
    """Strict check of the sparse decode path. A TEAL threshold is a discontinuity, so whole-model
    comparisons drift; here every stage of every block (qkv projection, attention on the packed
    pages, o_proj, norm, fused gate/up, down_proj) is fed exactly the tensors the HF + oracle-hook +
    oracle-cache run saw at that point of a decode step and must reproduce HF's next tensor."""
    from leankv_b200 import _native

    model = _hf_model(scale=2.0)
    gen = torch.Generator().manual_seed(5)
    prompt = torch.randint(0, 512, (41,), generator=gen).tolist()
    T = len(prompt)
    engine = DecodeEngine.from_hf(model, max_seq_len=128)
    engine.fused_norm = False            # keep the normed row as a buffer of its own so it can be compared
    thresholds = engine.calibrate_thresholds(prompt, 0.4)
    cache = OracleCache(model.config.num_hidden_layers, _dev())
    cap, hooks = {}, []

    def grab(key, pick):
        return lambda m, a, o=None: cap.__setitem__(key, pick(a, o).detach().clone().reshape(-1))

    with torch.no_grad():
        out = model(torch.tensor([prompt], device=_dev()), past_key_values=cache, use_cache=True)
        tok = int(out.logits[0, -1].float().argmax())
        for l, layer in enumerate(model.model.layers):
            for p in PROJ_NAMES:
                mod = getattr(layer.self_attn if p in ("q_proj", "k_proj", "v_proj", "o_proj") else layer.mlp, p)
                # record the raw input first, then let the oracle hook sparsify it
                hooks.append(mod.register_forward_pre_hook(grab((l, p, "in"), lambda a, o: a[0])))
                hooks.append(mod.register_forward_pre_hook(
                    lambda m, a, t=thresholds[l][p]: (oteal.sparsify(a[0], t),) + a[1:]))
                hooks.append(mod.register_forward_hook(grab((l, p, "out"), lambda a, o: o)))
            hooks.append(layer.register_forward_pre_hook(
                lambda m, a, kw, l=l: cap.__setitem__((l, "h_in"), (a[0] if a else kw["hidden_states"]).detach().clone().reshape(-1)),
                with_kwargs=True))
            hooks.append(layer.register_forward_hook(
                lambda m, a, o, l=l: cap.__setitem__((l, "h_out"), (o[0] if isinstance(o, tuple) else o).detach().clone().reshape(-1))))
        model(torch.tensor([[tok]], device=_dev()), past_key_values=cache, use_cache=True)
    for h in hooks:
        h.remove()

    lib = _native.lib()
    n_pages = (T + 15) // 16
    indptr = torch.tensor([0, n_pages], dtype=torch.int32, device=_dev())
    start = torch.zeros(1, dtype=torch.int32, device=_dev())
    report = {}
    for l in range(model.config.num_hidden_layers):
        k_hist, v_hist = cache.raw[l][0]                      # prompt k (after rope) and v, [1, nkv, T, 128]
        k_hist, v_hist = k_hist.half().contiguous(), v_hist.half().contiguous()
        engine.pools[l].zero_()
        _native.check(lib.leankv_tq_pool_append(k_hist.data_ptr(), v_hist.data_ptr(), 1, engine.nkv, T,
                                                engine.Pi_k[l].data_ptr(), engine.Pi_v[l].data_ptr(),
                                                engine.bounds.data_ptr(), engine.pools[l].data_ptr(),
                                                engine.max_pages, indptr.data_ptr(),
                                                engine.page_indices.data_ptr(), start.data_ptr(),
                                                torch.cuda.current_stream().cuda_stream), "pool_append")
        engine.state.copy_(torch.tensor([T, 1, 0, T // 16 + 1, T % 16 + 1, T, 0, 0], dtype=torch.int32))
        engine.h.copy_(cap[(l, "h_in")])
        engine._norm(None, engine.w["layers"][l]["ln1"])
        torch.cuda.synchronize()
        report[(l, "x1")] = rel_l2(engine.x.float().cpu(), cap[(l, "q_proj", "in")].float().cpu())
        engine.x.copy_(cap[(l, "q_proj", "in")])

        def probe(stage, l=l):
            """Compare the buffer this stage wrote with HF's tensor, then overwrite it with HF's so that
            the next stage starts from identical inputs (same mask, bit for bit)."""
            torch.cuda.synchronize()
            if stage == "qkv":
                want = torch.cat([cap[(l, p, "out")] for p in ("q_proj", "k_proj", "v_proj")])
                buf = engine.qkv
            elif stage == "attn":
                want, buf = cap[(l, "o_proj", "in")], engine.attn
            elif stage == "o":
                want, buf = cap[(l, "o_proj", "out")], engine.o
            elif stage == "x":
                want, buf = cap[(l, "gate_proj", "in")], engine.x
            elif stage == "mlp_h":
                want, buf = cap[(l, "down_proj", "in")], engine.mlp_h
            else:
                want, buf = cap[(l, "down_proj", "out")], engine.down
            report[(l, stage)] = rel_l2(buf.float().cpu(), want.float().cpu())
            buf.copy_(want)

        engine._layer_launches(l, probe)
        torch.cuda.synchronize()
        report[(l, "h_out")] = rel_l2(engine.h.float().cpu(), cap[(l, "h_out")].float().cpu())
    print("per-stage rel-L2 on identical inputs:", {k: f"{v:.1e}" for k, v in report.items()})
    for (l, stage), err in report.items():
        # attention: the new token's k/v codes come from this path's own projection output (copied
        # from HF here, so identical) -> only fp16/fp32 rounding remains everywhere
        assert err < (3e-3 if stage == "attn" else 1.5e-3), (l, stage, err)


def test_fused_norm_matches_separate_norm_launches():
    """RMSNorm fused into the projection kernels sums the squares in another order than the stand-alone
    kernel, so the two paths agree to rounding, not bit for bit."""
    model = _hf_model(scale=1.0)
    prompt = list(range(11, 70))
    runs = []
    for fused in (True, False):
        eng = DecodeEngine.from_hf(model, max_seq_len=128)
        eng.fused_norm = fused
        toks, logits = _engine_run(eng, prompt, 10, follow_tokens=[5, 9, 200, 31, 77, 8, 400, 3, 12])
        runs.append(logits)
    errs = [rel_l2(a, b) for a, b in zip(*runs)]
    print("fused vs separate norm rel-L2:", [f"{e:.1e}" for e in errs])
    assert max(errs) < 5e-3


def test_fused_post_kernel_is_bit_identical_to_separate_launches():
    model = _hf_model(scale=2.0)
    prompt = list(range(7, 60))
    runs = []
    for fused in (True, False):
        eng = DecodeEngine.from_hf(model, max_seq_len=128)
        eng.fused_post = fused
        eng.calibrate_thresholds(prompt, 0.4)
        toks, logits = _engine_run(eng, prompt, 12)
        runs.append((toks, logits, [p.clone() for p in eng.pools]))
    assert runs[0][0] == runs[1][0]
    assert all(torch.equal(a, b) for a, b in zip(runs[0][1], runs[1][1]))
    assert all(torch.equal(a, b) for a, b in zip(runs[0][2], runs[1][2]))


def test_prefill_in_chunks_over_packed_pages_matches_whole_prompt_and_dense_attention():
    """Chunked prefill (every chunk quantized first, then attending to the packed pages) against the
    whole prompt in one pass and against the route that de-quantizes and calls library attention."""
    engine = DecodeEngine.from_hf(_hf_model(2, scale=2.0), max_seq_len=256)
    prompt = list(range(3, 3 + 200))
    engine.prefill(prompt, attention="dense")
    dense = engine.prefill_logits.float().clone()
    pool_dense = engine.pools[0].clone()
    engine.prefill(prompt)
    whole = engine.prefill_logits.float().clone()
    engine.prefill(prompt, chunk=64)
    chunked = engine.prefill_logits.float().clone()
    engine.prefill(prompt)          # the workspace has served chunks of another length in between
    assert torch.equal(engine.prefill_logits.float(), whole)
    assert rel_l2(whole.cpu(), dense.cpu()) < 2e-2
    assert rel_l2(chunked.cpu(), whole.cpu()) < 2e-2
    # layer 0's keys and values do not depend on attention at all: identical pools
    assert torch.equal(engine.pools[0], pool_dense)
    with pytest.raises(ValueError):
        engine.prefill(prompt, chunk=64, attention="dense")


def test_sharded_argmax_with_a_single_rank_exchanging_with_itself():
    """``leankv_decode_end_sharded`` on one GPU: the rank's slice is the whole vocabulary shifted by an
    offset; the token is the arg-max (lowest index on ties), position / step / history advance and the
    exchange's epoch moves on by one per call."""
    import ctypes

    from leankv_b200 import _native
    from leankv_b200.peer_exchange import PeerExchange

    dev = _dev()
    lib = _native.lib()
    ex = PeerExchange(dev, 0, 1, None, n_slots=3, max_cols=256)
    gen = torch.Generator().manual_seed(4)
    logits = torch.randn(4096, generator=gen).half().to(dev)
    logits[1234] = 9.0
    logits[3000] = 9.0                      # a tie: the lower index wins
    token = torch.zeros(1, dtype=torch.int64, device=dev)
    history = torch.zeros(16, dtype=torch.int64, device=dev)
    state = torch.zeros(8, dtype=torch.int32, device=dev)
    state[0] = 41
    st = torch.cuda.current_stream().cuda_stream
    for call in range(3):
        rc = lib.leankv_decode_end_sharded(logits.data_ptr(), 4096, 32768, token.data_ptr(), history.data_ptr(), 16,
                                           state.data_ptr(), ctypes.byref(ex.c), 2, st)
        _native.check(rc, "decode_end_sharded")
        torch.cuda.synchronize()
        assert int(token.item()) == 32768 + 1234
        assert int(ex.epoch.item()) == 2 + call
        assert state[:2].tolist() == [42 + call, 1 + call]
        assert int(history[call].item()) == 32768 + 1234
    assert not ex.timed_out()
    ex.close()
