"""Generates the golden fixtures in this directory from the REFERENCE implementation.

Run once in a container where the reference project is importable:

    python tests/golden/make_golden.py /path/to/leankv-reference

It imports the reference's own modules (redirecting its codebook cache so that nothing is
written into the reference tree), feeds them the seeded inputs of ``leankv_b200.workloads``
and small ragged cases, and stores inputs' seeds + the reference's outputs. The tests then
pin the CPU oracle (``oracle/``) and the CUDA kernels against these files. Fixtures hold
reference OUTPUTS only (plus small inputs); no reference source is copied.
"""

import hashlib
import json
import os
import sys
import tempfile

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)


def main(ref_root: str) -> None:
    sys.path.insert(0, ref_root)
    import leankv.turboquant.codebook as ref_cb

    ref_cb._CODEBOOK_DIR = tempfile.mkdtemp(prefix="leankv_ref_codebooks_")
    from leankv.teal.sparse_fns import (SparsifyFn, compute_threshold_for_sparsity,
                                        compute_threshold_from_histogram)
    from leankv.turboquant.cache import TurboQuantCache
    from leankv.turboquant.quantizer import TurboQuantMSE, _pack_indices, _unpack_indices
    from leankv.turboquant.rotation import generate_rotation_matrix

    from leankv_b200 import workloads

    torch.set_num_threads(8)
    dev = torch.device("cpu")

    # 1. codebooks (doubles, reference JSON schema)
    books = {str(b): ref_cb.compute_lloyd_max_codebook(128, b) for b in (1, 2, 3, 4)}
    with open(os.path.join(HERE, "codebooks_d128.json"), "w") as f:
        json.dump(books, f, indent=1)

    # 2. rotations for the seeds a 32-layer cache uses (42 .. 105)
    rot = {}
    for seed in range(42, 106):
        Pi = generate_rotation_matrix(128, dev, torch.float32, seed=seed)
        rot[str(seed)] = {"sha256": hashlib.sha256(Pi.numpy().tobytes()).hexdigest(),
                          "row0_head": Pi[0, :4].tolist()}
    with open(os.path.join(HERE, "rotations_d128.json"), "w") as f:
        json.dump(rot, f, indent=1)

    # 3. TEAL: thresholds, masks and GEMV outputs
    out = {}
    c1 = workloads.sparse_gemv_case()                      # config 1
    t1 = compute_threshold_for_sparsity(c1.x, 0.4)
    xs = SparsifyFn(t1)(c1.x)
    out["c1_threshold"] = np.float64(t1)
    out["c1_n_active"] = np.int64((xs != 0).sum().item())
    out["c1_y_fp16"] = torch.nn.functional.linear(xs, c1.weight).numpy()
    out["c1_y_fp32"] = torch.nn.functional.linear(xs.float(), c1.weight.float()).numpy()
    c2 = workloads.swiglu_case()                           # config 2
    t2 = compute_threshold_for_sparsity(c2.x, 0.4)
    xs2 = SparsifyFn(t2)(c2.x)
    g = torch.nn.functional.linear(xs2, c2.w_gate)
    u = torch.nn.functional.linear(xs2, c2.w_up)
    out["c2_threshold"] = np.float64(t2)
    out["c2_n_active"] = np.int64((xs2 != 0).sum().item())
    out["c2_y_fp16"] = (torch.nn.functional.silu(g) * u).numpy()
    g32 = torch.nn.functional.linear(xs2.float(), c2.w_gate.float())
    u32 = torch.nn.functional.linear(xs2.float(), c2.w_up.float())
    out["c2_y_fp32"] = (torch.nn.functional.silu(g32) * u32).numpy()
    # ragged small cases: (N, Z, sparsity, seed); inputs are regenerated from the seed
    small = [(8, 5, 0.4, 11), (264, 33, 0.0, 12), (520, 1000, 0.9, 13), (1024, 4096, 0.5, 14),
             (4096, 4096, 0.4, 15), (16, 1, 0.0, 16), (2048, 2500, 1.0, 17)]
    out["small_cases"] = np.array(small, dtype=np.float64)
    for i, (n, z, s, seed) in enumerate(small):
        c = workloads.sparse_gemv_case(int(n), int(z), s, int(seed))
        t = compute_threshold_for_sparsity(c.x, s)
        xm = SparsifyFn(t)(c.x)
        out[f"small{i}_threshold"] = np.float64(t)
        out[f"small{i}_mask"] = (xm != 0).numpy() if t > 0 else np.ones_like(c.x.numpy(), dtype=bool)
        out[f"small{i}_y_fp16"] = torch.nn.functional.linear(xm, c.weight).numpy()
        out[f"small{i}_y_fp32"] = torch.nn.functional.linear(xm.float(), c.weight.float()).numpy()
    # histogram thresholds
    hgen = torch.Generator().manual_seed(5)
    acts = torch.randn(20000, generator=hgen).abs()
    counts, edges = torch.histogram(acts, bins=200)
    out["hist_counts"] = counts.numpy()
    out["hist_edges"] = edges.numpy()
    out["hist_targets"] = np.array([0.0, 0.003, 0.3, 0.4, 0.5, 0.9, 0.999])
    out["hist_thresholds"] = np.array(
        [compute_threshold_from_histogram(counts, edges, float(s)) for s in out["hist_targets"]])
    np.savez_compressed(os.path.join(HERE, "teal.npz"), **out)

    # 4. TurboQuant: quantize / dequantize / attention on a small config-3-shaped case
    tq = {}
    kv = workloads.kv_case(batch=2, n_q_heads=8, n_kv_heads=2, context=70, seed=3)
    qk = TurboQuantMSE(128, 3, dev, torch.float32, seed=42)
    qv = TurboQuantMSE(128, 3, dev, torch.float32, seed=43)
    tq["centroids"] = qk.centroids.numpy()
    tq["decision_boundaries"] = qk.decision_boundaries.numpy()
    for name, quant, x in (("k", qk, kv.k), ("v", qv, kv.v)):
        qq = quant.quantize(x.float())
        tq[f"{name}_indices"] = qq.indices.numpy()
        tq[f"{name}_norms"] = qq.norms.numpy()
        tq[f"{name}_dequant"] = quant.dequantize(qq).numpy()
        # the rotated coordinates themselves, to measure distance to the boundaries
        unit = x.float() / (x.float().norm(dim=-1, keepdim=True) + 1e-10)
        tq[f"{name}_rotated"] = torch.matmul(unit, quant.Pi.T).numpy()
        # config-3 semantics: norms rounded to fp16 before reconstruction
        q16 = qq._replace(norms=qq.norms.half().float())
        tq[f"{name}_dequant_fp16norm_half"] = quant.dequantize(q16).half().numpy()
    # attention the way a decode step sees it: fp16 K_hat/V_hat (cache.py:176-181), GQA, fp32 softmax
    k_hat = torch.from_numpy(tq["k_dequant_fp16norm_half"]).float()
    v_hat = torch.from_numpy(tq["v_dequant_fp16norm_half"]).float()
    rep = kv.q.shape[1] // k_hat.shape[1]
    kk = k_hat.repeat_interleave(rep, dim=1)
    vv = v_hat.repeat_interleave(rep, dim=1)
    lengths = [70, 37]
    scores = torch.einsum("bhd,bhtd->bht", kv.q.float(), kk) * (128 ** -0.5)
    mask = torch.arange(70).unsqueeze(0) >= torch.tensor(lengths).unsqueeze(1)
    scores = scores.masked_fill(mask.unsqueeze(1), float("-inf"))
    tq["attn_lengths"] = np.array(lengths)
    tq["attn_out"] = torch.einsum("bht,bhtd->bhd", torch.softmax(scores, -1), vv).numpy()
    # other bit widths on a handful of vectors
    xs_small = kv.k[0, 0, :9].float()
    for bits in (1, 2, 4):
        qb = TurboQuantMSE(128, bits, dev, torch.float32, seed=7)
        qq = qb.quantize(xs_small)
        tq[f"b{bits}_indices"] = qq.indices.numpy()
        tq[f"b{bits}_norms"] = qq.norms.numpy()
        tq[f"b{bits}_dequant"] = qb.dequantize(qq).numpy()
    # pack / unpack of arbitrary codes with ragged length
    pgen = torch.Generator().manual_seed(9)
    for bits in (1, 2, 3, 4, 6):
        codes = torch.randint(0, 2 ** bits, (3, 13), generator=pgen)
        packed = _pack_indices(codes, bits)
        tq[f"pack_b{bits}_codes"] = codes.numpy()
        tq[f"pack_b{bits}_packed"] = packed.numpy()
        assert torch.equal(_unpack_indices(packed, bits, 13), codes)
    np.savez_compressed(os.path.join(HERE, "turboquant.npz"), **tq)

    # 5. TurboQuantCache.update trace: 2 layers, hot buffer 4, prefill 7 tokens + 6 single steps
    cgen = torch.Generator().manual_seed(21)
    cache = TurboQuantCache(bits=3, head_dim=128, num_layers=2, hot_buffer_size=4, device=dev,
                            dtype=torch.float16, seed=42)
    steps = [7, 1, 1, 1, 1, 1, 1]
    trace = {"steps": np.array(steps)}
    for si, t_new in enumerate(steps):
        for layer in range(2):
            k = torch.randn(2, 2, t_new, 128, generator=cgen).half()
            v = torch.randn(2, 2, t_new, 128, generator=cgen).half()
            K, V = cache.update(k, v, layer)
            trace[f"k_in_{si}_{layer}"] = k.numpy()
            trace[f"v_in_{si}_{layer}"] = v.numpy()
            if si == len(steps) - 1:
                trace[f"K_out_{layer}"] = K.numpy()
                trace[f"V_out_{layer}"] = V.numpy()
    trace["seq_length"] = np.int64(cache.get_seq_length(0))
    trace["cold_length"] = np.int64(cache._cold_lengths[0])
    trace["compression_ratio"] = np.float64(cache.get_compression_ratio())
    trace["compressed_bytes"] = np.int64(cache.get_compressed_memory_bytes())
    np.savez_compressed(os.path.join(HERE, "cache_trace.npz"), **trace)
    print("golden fixtures written to", HERE)


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: python tests/golden/make_golden.py <path to a checkout of asmit383/leankv>")
    main(sys.argv[1])
