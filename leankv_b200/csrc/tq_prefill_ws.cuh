// Warp-specialised form of the prefill attention on the fifth-generation tensor cores: the rotated query tile
// and the probabilities live in tensor memory as the A operands of the two products, so the only operands
// read from shared memory are the de-quantized keys and values.
//
// One CTA per SM (512 tensor-memory columns), 13 warps:
//   warps 0-3   softmax: thread t = row t = accumulator lane t. Stage Q'' (fp16 high and low halves) into tensor
//               memory once; per block read S, apply norm / mask / running maximum, rescale O when the lazy
//               maximum moved, store the fp16 probabilities (times value norm) into tensor memory.
//   warps 4-7   keys: one 32-code unit per thread and block -> K tile (two buffers)
//   warps 8-11  values: one unit per thread and block, 4-lane transpose -> V tile (two buffers); the block's norms
//   warp 12     thread 0 issues the page copies and the MMAs: S(b+1) goes out before O += P(b) V(b)
// The roles meet only through mbarriers (bounded waits; a role that gives up leaves its loop, the others follow
// through their own limits): page copies (4 stages) -> keys ready / values ready (2 each) -> S done (2, commit) ->
// probabilities ready -> PV done (2, commit). Every waiter sees every phase of a barrier it waits on in order.
// Same page ranges, partial results and status bits as tq_prefill_t5_kernel.
// (included by tq_attn.cu after tq_prefill_kernel.cuh, inside namespace leankv::{anonymous})
#pragma once

constexpr int kWsThreads = 416;
constexpr int kWsIssuer = 384;
constexpr int kWsStages = 4;
constexpr uint32_t kWsTmemCols = 512;
constexpr uint32_t kWsColQh = 0, kWsColQl = 64, kWsColS = 128, kWsColP = 192, kWsColO = 256;
// barrier indices
constexpr int kWsBarRaw = 0, kWsBarK = 4, kWsBarV = 6, kWsBarP = 8, kWsBarS = 9, kWsBarPV = 11, kWsBarQ = 13, kWsBars = 14;
// more than half of an SM's shared memory, so that one CTA (and its 512 columns) owns the SM
constexpr size_t kWsSmemBytes = 120 * 1024;

__global__ void __launch_bounds__(kWsThreads, 1) tq_prefill_ws_kernel(const PrefillParams p) {
    extern __shared__ __align__(1024) uint8_t ws_smem[];
    uint8_t* s_k = ws_smem;                                            // [2] K tiles  [token][coord]
    uint8_t* s_v = s_k + 2 * (size_t)kT5KTileBytes;                    // [2] V tiles  [coord][token]
    uint8_t* s_raw = s_v + 2 * (size_t)kDim * kT5N * 2;                // [stages][page of the block][K chunk | V chunk]
    float* s_kn = reinterpret_cast<float*>(s_raw + (size_t)kWsStages * kT5Blk * 2 * kChunkBytes);   // [block & 3][32]
    float* s_vn = s_kn + 4 * kT5N;
    uint64_t* s_bar = reinterpret_cast<uint64_t*>(s_vn + 4 * kT5N);
    uint32_t* s_tmem = reinterpret_cast<uint32_t*>(s_bar + kWsBars);

    const int tid = threadIdx.x, warp = tid >> 5;
    const int H = p.H, Hq = H * kGroup;
    const int n_tiles = (p.T + 31) / 32;
    const int tile = n_tiles - 1 - (int)blockIdx.x;
    const int kvh = blockIdx.y;
    const int tok0 = tile * 32;
    const int last_tok = min(tok0 + 32, p.T) - 1;
    const int n_all = (p.start_pos + last_tok) / kPage + 1;
    const int pg_lo = split_begin(p, n_all, blockIdx.z);
    const int n_pg = split_begin(p, n_all, blockIdx.z + 1) - pg_lo;
    const int n_blk = (n_pg + kT5Blk - 1) / kT5Blk;

    const uint32_t bar0 = smem_u32(s_bar);
    auto bar = [&](int idx) { return bar0 + 8u * (uint32_t)idx; };
    // block b is use number b / 4 of its raw stage and b / 2 of every two-buffer barrier: those uses' phase parities
    auto par4 = [](int b) { return (uint32_t)((b >> 2) & 1); };
    auto par2 = [](int b) { return (uint32_t)((b >> 1) & 1); };
    int where = 0;
    bool failed = false;
    bool bad_page = false;
    auto wait = [&](int idx, uint32_t parity, int why) -> bool {
        if (umma::bar_wait(bar(idx), parity)) return true;
        failed = true;
        where |= why;
        return false;
    };

    // the same, with the outcome made common to the warp (roles that run warp-wide instructions must leave together)
    auto wait_warp = [&](int idx, uint32_t parity, int why) -> bool {
        const bool ok = __all_sync(0xffffffffu, wait(idx, parity, why));
        if (!ok) failed = true;
        return ok;
    };

    if (warp == 0) umma::tmem_alloc_n(smem_u32(s_tmem), kWsTmemCols);
    if (tid == 0) {
        for (int i = 0; i < kWsStages; ++i) umma::bar_init_n(bar(kWsBarRaw + i), 1);
        for (int i = 0; i < 2; ++i) {
            umma::bar_init_n(bar(kWsBarK + i), 128);
            umma::bar_init_n(bar(kWsBarV + i), 128);
            umma::bar_init_n(bar(kWsBarS + i), 1);
            umma::bar_init_n(bar(kWsBarPV + i), 1);
        }
        umma::bar_init_n(bar(kWsBarP), 128);
        umma::bar_init_n(bar(kWsBarQ), 128);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    pdl_begin();
    umma::fence_before_sync();
    __syncthreads();
    umma::fence_after_sync();
    const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(s_tmem);
    const uint32_t tmem_o = tmem_base + kWsColO;

    if (warp == 12) {
        // ------------------------------------------------------------------ issuing thread
        if (tid == kWsIssuer) {
            const size_t page_stride = (size_t)2 * H * kChunkBytes, kv_stride = (size_t)H * kChunkBytes;
            const uint8_t* pool_kvh = p.pool + (size_t)kvh * kChunkBytes;
            int next_id[kT5Blk] = {0, 0};
            int n_issued = 0;
            auto load_ids = [&](int blk) {
#pragma unroll
                for (int i = 0; i < kT5Blk; ++i)
                    next_id[i] = blk * kT5Blk + i < n_pg ? p.seq_pages[pg_lo + blk * kT5Blk + i] : 0;
            };
            auto issue_pages = [&](int blk) {                // calls come in block order
                const int st = blk % kWsStages;
                const int n_here = min(kT5Blk, n_pg - blk * kT5Blk);
                mbar_expect_tx(bar(kWsBarRaw + st), (uint32_t)n_here * 2 * kChunkBytes);
#pragma unroll
                for (int i = 0; i < kT5Blk; ++i) {
                    if (i >= n_here) break;
                    int id = next_id[i];
                    if (id < 0 || id >= p.n_pages) {
                        id = 0;
                        bad_page = true;
                    }
                    const uint8_t* src = pool_kvh + (size_t)id * page_stride;
                    const uint32_t dst = smem_u32(s_raw + ((size_t)st * kT5Blk + i) * 2 * kChunkBytes);
                    bulk_g2s(dst, src, kChunkBytes, bar(kWsBarRaw + st));
                    bulk_g2s(dst + kChunkBytes, src + kv_stride, kChunkBytes, bar(kWsBarRaw + st));
                }
                n_issued = blk + 1;
                load_ids(blk + 1);
            };
            auto issue_scores = [&](int b) {                 // S(b) = Q''_h K^T + Q''_l K^T into score buffer b & 1
                const uint32_t kb = smem_u32(s_k) + (uint32_t)(b & 1) * kT5KTileBytes;
                const uint32_t ts = tmem_base + kWsColS + (uint32_t)(b & 1) * kT5N;
#pragma unroll
                for (int ks = 0; ks < kDim / 16; ++ks) {
                    const uint32_t off = (uint32_t)ks * 2 * umma::kLbo;
                    umma::mma_f16_ts(ts, tmem_base + kWsColQh + 8 * ks, umma::desc(kb + off), umma::idesc_n(kT5N), ks == 0 ? 0u : 1u);
                    umma::mma_f16_ts(ts, tmem_base + kWsColQl + 8 * ks, umma::desc(kb + off), umma::idesc_n(kT5N), 1u);
                }
                umma::commit(bar(kWsBarS + (b & 1)));
            };
            load_ids(0);
            for (int blk = 0; blk < min(kWsStages, n_blk); ++blk) issue_pages(blk);
            bool ok = wait(kWsBarQ, 0, kT5WhereScores);
            if (ok && n_blk > 0) {
                ok = wait(kWsBarK + 0, 0, kT5WherePages);
                umma::fence_after_sync();
                if (ok) issue_scores(0);
            }
            for (int blk = 0; blk < n_blk && ok; ++blk) {
                if (blk + 1 < n_blk) {
                    ok = wait(kWsBarK + ((blk + 1) & 1), par2(blk + 1), kT5WherePages);
                    if (!ok) break;
                    umma::fence_after_sync();
                    issue_scores(blk + 1);
                }
                ok = wait(kWsBarP, (uint32_t)(blk & 1), kT5WhereScores) && wait(kWsBarV + (blk & 1), par2(blk), kT5WherePages);
                if (!ok) break;
                umma::fence_after_sync();
                const uint32_t vb = smem_u32(s_v) + (uint32_t)(blk & 1) * (kDim * kT5N * 2);
#pragma unroll
                for (int kt = 0; kt < kT5N / 16; ++kt) {
                    const uint32_t off = (uint32_t)kt * 2 * umma::kLbo;
                    umma::mma_f16_ts(tmem_o, tmem_base + kWsColP + 8 * kt, umma::desc_k(vb + off, kT5KChunksTok),
                                     umma::idesc_n(kDim), (blk == 0 && kt == 0) ? 0u : 1u);
                }
                umma::commit(bar(kWsBarPV + (blk & 1)));
                if (blk + kWsStages < n_blk) issue_pages(blk + kWsStages);   // keys and values of block blk are both out of the stage
            }
            if (failed) {
                // give page copies that may still be in flight a bounded chance to land in this CTA's shared memory
                for (int b = max(0, n_issued - kWsStages); b < n_issued; ++b) umma::bar_wait(bar(kWsBarRaw + b % kWsStages), par4(b));
            }
        }
    } else if (warp >= 8) {
        // ------------------------------------------------------------------ values (and the block's norms)
        const int t = tid - 256, pgi = t >> 6, ui = t & 63;
        for (int blk = 0; blk < n_blk; ++blk) {
            if (!wait_warp(kWsBarRaw + blk % kWsStages, par4(blk), kT5WherePages)) break;
            if (blk >= 2 && !wait_warp(kWsBarPV + (blk & 1), par2(blk - 2), kT5WhereValues)) break;   // O += P V of block blk - 2 read this tile
            const uint8_t* chunk = s_raw + ((size_t)(blk % kWsStages) * kT5Blk + pgi) * 2 * kChunkBytes + kChunkBytes;
            const Unit u = load_unit(reinterpret_cast<const uint32_t*>(chunk), ui);
            uint32_t h2[16];
#pragma unroll
            for (int w = 0; w < 4; ++w) {
                const uint32_t sa = u.s[w], sb = sa >> 16;
                const uint32_t la = __byte_perm(p.tl0, p.tl1, sa), ha = __byte_perm(p.th0, p.th1, sa);
                const uint32_t lb = __byte_perm(p.tl0, p.tl1, sb), hb = __byte_perm(p.th0, p.th1, sb);
                h2[4 * w + 0] = __byte_perm(la, ha, 0x5140);
                h2[4 * w + 1] = __byte_perm(la, ha, 0x7362);
                h2[4 * w + 2] = __byte_perm(lb, hb, 0x5140);
                h2[4 * w + 3] = __byte_perm(lb, hb, 0x7362);
            }
            // register i = the unit's two tokens of coordinate 16 grp + i; lanes 4n .. 4n+3 hold the 8 tokens of a
            // 16-byte piece: a 4 x 4 transpose between them leaves lane pl with the whole piece of coordinates 4j + pl
            uint8_t* vt = s_v + (size_t)(blk & 1) * (kDim * kT5N * 2);
            const int grp = (ui & 31) >> 2, pl = ui & 3, half = ui >> 5;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                uint32_t* a = h2 + 4 * j;
#pragma unroll
                for (int c = 0; c < 4; c += 2) {
                    const uint32_t send = (pl & 1) ? a[c] : a[c + 1];
                    const uint32_t got = __shfl_xor_sync(0xffffffffu, send, 1);
                    if (pl & 1) a[c] = got; else a[c + 1] = got;
                }
#pragma unroll
                for (int c = 0; c < 2; ++c) {
                    const uint32_t send = (pl & 2) ? a[c] : a[c + 2];
                    const uint32_t got = __shfl_xor_sync(0xffffffffu, send, 2);
                    if (pl & 2) a[c] = got; else a[c + 2] = got;
                }
                *reinterpret_cast<uint4*>(vt + umma::offset_k(16 * grp + 4 * j + pl, 2 * pgi + half, kT5KChunksTok)) =
                    make_uint4(a[0], a[1], a[2], a[3]);
            }
            if (t < 2 * kT5N) {                              // key norms (t < 32) and value norms, times 1 / alpha; 0 beyond the range
                const int j = t & (kT5N - 1), is_v = t >> 5, pj = j >> 4;
                float v = 0.f;
                if (blk * kT5Blk + pj < n_pg) {
                    const uint8_t* rw = s_raw + ((size_t)(blk % kWsStages) * kT5Blk + pj) * 2 * kChunkBytes + (is_v ? kChunkBytes : 0);
                    v = __half2float(reinterpret_cast<const __half*>(rw + kNormOffsetBytes)[j & 15]) * p.inv_alpha;
                }
                (is_v ? s_vn : s_kn)[(blk & 3) * kT5N + j] = v;
            }
            umma::fence_operands();
            umma::bar_arrive(bar(kWsBarV + (blk & 1)));
        }
    } else if (warp >= 4) {
        // ------------------------------------------------------------------ keys
        const int t = tid - 128, pgi = t >> 6, ui = t & 63;
        const int ktok = ui & 15, kq = ui >> 4;              // 8 consecutive lanes = 8 consecutive tokens of one quarter
        for (int blk = 0; blk < n_blk; ++blk) {
            if (!wait_warp(kWsBarRaw + blk % kWsStages, par4(blk), kT5WherePages)) break;
            if (blk >= 2 && !wait_warp(kWsBarS + (blk & 1), par2(blk - 2), kT5WhereScores)) break;    // S of block blk - 2 read this tile
            const uint8_t* chunk = s_raw + ((size_t)(blk % kWsStages) * kT5Blk + pgi) * 2 * kChunkBytes;
            const Unit u = load_unit(reinterpret_cast<const uint32_t*>(chunk), 4 * ktok + kq);
            uint32_t h2[16];
#pragma unroll
            for (int w = 0; w < 4; ++w) {
                const uint32_t sa = u.s[w], sb = sa >> 16;
                const uint32_t la = __byte_perm(p.tl0, p.tl1, sa), ha = __byte_perm(p.th0, p.th1, sa);
                const uint32_t lb = __byte_perm(p.tl0, p.tl1, sb), hb = __byte_perm(p.th0, p.th1, sb);
                h2[4 * w + 0] = __byte_perm(la, ha, 0x5140);
                h2[4 * w + 1] = __byte_perm(la, ha, 0x7362);
                h2[4 * w + 2] = __byte_perm(lb, hb, 0x5140);
                h2[4 * w + 3] = __byte_perm(lb, hb, 0x7362);
            }
            uint8_t* kt = s_k + (size_t)(blk & 1) * kT5KTileBytes;
            const int trow = 16 * pgi + ktok, k8 = 4 * kq;
#pragma unroll
            for (int q = 0; q < 4; ++q)
                *reinterpret_cast<uint4*>(kt + umma::offset(trow, k8 + q)) = make_uint4(h2[4 * q], h2[4 * q + 1], h2[4 * q + 2], h2[4 * q + 3]);
            umma::fence_operands();
            umma::bar_arrive(bar(kWsBarK + (blk & 1)));
        }
    }

    // ---------------------------------------------------------------------- softmax rows (warps 0-3)
    const int row = tid & 127, lane0 = 32 * (warp & 3);
    const int tok = tok0 + (row >> 2), head = row & 3;
    const int qpos = p.start_pos + tok;
    float m_ref = kNoRef, l_run = 0.f;
    int n_pv = 0;
    if (warp < 4) {
        // the row's query: rotated, scaled, fp16 high and low halves, two per column, into tensor memory
        const float* qsrc = p.qprime + ((size_t)min(tok, p.T - 1) * Hq + (size_t)kvh * kGroup + head) * kDim;
        const float qs = tok < p.T ? p.qscale : 0.f;
#pragma unroll
        for (int c0 = 0; c0 < kDim; c0 += 64) {
            uint32_t hi[32], lo[32];
#pragma unroll
            for (int e = 0; e < 16; ++e) {
                const float4 x = *reinterpret_cast<const float4*>(qsrc + c0 + 4 * e);
                const float v0 = x.x * qs, v1 = x.y * qs, v2 = x.z * qs, v3 = x.w * qs;
                const __half2 h01 = __floats2half2_rn(v0, v1), h23 = __floats2half2_rn(v2, v3);
                const float2 f01 = __half22float2(h01), f23 = __half22float2(h23);
                const __half2 l01 = __floats2half2_rn(v0 - f01.x, v1 - f01.y), l23 = __floats2half2_rn(v2 - f23.x, v3 - f23.y);
                hi[2 * e] = *reinterpret_cast<const uint32_t*>(&h01);
                hi[2 * e + 1] = *reinterpret_cast<const uint32_t*>(&h23);
                lo[2 * e] = *reinterpret_cast<const uint32_t*>(&l01);
                lo[2 * e + 1] = *reinterpret_cast<const uint32_t*>(&l23);
            }
            umma::st32(hi, tmem_base + kWsColQh, lane0, c0 / 2);
            umma::st32(lo, tmem_base + kWsColQl, lane0, c0 / 2);
        }
        umma::fence_before_sync();
        umma::bar_arrive(bar(kWsBarQ));

        for (int blk = 0; blk < n_blk; ++blk) {
            // the block's norms come with its values; its scores with the MMA group's commit
            if (!wait_warp(kWsBarV + (blk & 1), par2(blk), kT5WherePages)) break;
            if (!wait_warp(kWsBarS + (blk & 1), par2(blk), kT5WhereScores)) break;
            umma::fence_after_sync();
            uint32_t sv[32];
            umma::ld32(sv, tmem_base + kWsColS + (uint32_t)(blk & 1) * kT5N, lane0, 0);
            const int kbase = (pg_lo + blk * kT5Blk) * kPage;
            const int n_tok_here = min(kT5Blk, n_pg - blk * kT5Blk) * kPage;     // tokens of this block that lie in the range
            // a whole block at or below the tile's first query position needs no mask (CTA-uniform)
            const bool full = n_tok_here == kT5N && kbase + kT5N - 1 <= p.start_pos + tok0;
            float sc[32];
            float bmax = kNoRef;
            {
                const float4* kn4 = reinterpret_cast<const float4*>(s_kn + (blk & 3) * kT5N);
#pragma unroll
                for (int j4 = 0; j4 < 8; ++j4) {
                    const float4 n = kn4[j4];
                    sc[4 * j4 + 0] = __uint_as_float(sv[4 * j4 + 0]) * n.x;
                    sc[4 * j4 + 1] = __uint_as_float(sv[4 * j4 + 1]) * n.y;
                    sc[4 * j4 + 2] = __uint_as_float(sv[4 * j4 + 2]) * n.z;
                    sc[4 * j4 + 3] = __uint_as_float(sv[4 * j4 + 3]) * n.w;
                }
                if (!full) {
#pragma unroll
                    for (int j = 0; j < 32; ++j)
                        if (!(j < n_tok_here && kbase + j <= qpos)) sc[j] = kNoRef;
                }
#pragma unroll
                for (int j = 0; j < 32; ++j) bmax = fmaxf(bmax, sc[j]);
            }
            // the reference only moves when the block exceeds it by more than the slack
            const bool move = bmax > m_ref + kT5Slack;
            const float m_new = move ? bmax : m_ref;
            const float f = move ? ex2_approx(m_ref - m_new) : 1.0f;
            m_ref = m_new;
            l_run *= f;
            uint32_t pw[16];                                  // probabilities (at most 2^slack) times value norm, fp16 pairs
            {
                float sum = 0.f;
                const float4* vn4 = reinterpret_cast<const float4*>(s_vn + (blk & 3) * kT5N);
#pragma unroll
                for (int j4 = 0; j4 < 8; ++j4) {
                    const float4 n = vn4[j4];
                    float pr[4];
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const float x = sc[4 * j4 + e];
                        // a masked entry gives 0 (with no reference yet x - m_ref would be 0, hence the test)
                        pr[e] = (full || x > 0.5f * kNoRef) ? ex2_approx(x - m_ref) : 0.f;
                    }
                    sum += (pr[0] + pr[1]) + (pr[2] + pr[3]);
                    const __half2 a = __floats2half2_rn(pr[0] * n.x, pr[1] * n.y), b2 = __floats2half2_rn(pr[2] * n.z, pr[3] * n.w);
                    pw[2 * j4] = *reinterpret_cast<const uint32_t*>(&a);
                    pw[2 * j4 + 1] = *reinterpret_cast<const uint32_t*>(&b2);
                }
                l_run += sum;
            }
            // O += P V of the previous block reads P and writes O: it must be done before either is touched
            if (blk > 0) {
                if (!wait_warp(kWsBarPV + ((blk - 1) & 1), par2(blk - 1), kT5WhereValues)) break;
                umma::fence_after_sync();
                // rows of O are rescaled in tensor memory when the reference moved (all lanes of a warp take part;
                // lanes that did not move use factor 1)
                if (__any_sync(0xffffffffu, move)) {
#pragma unroll
                    for (int c0 = 0; c0 < kDim; c0 += 32) {
                        uint32_t ov[32];
                        umma::ld32(ov, tmem_o, lane0, c0);
#pragma unroll
                        for (int i = 0; i < 32; ++i) ov[i] = __float_as_uint(__uint_as_float(ov[i]) * f);
                        umma::st32(ov, tmem_o, lane0, c0);
                    }
                }
            }
            umma::st16(pw, tmem_base + kWsColP, lane0, 0);
            umma::fence_before_sync();
            umma::bar_arrive(bar(kWsBarP));
            n_pv = blk + 1;
        }
        if (!failed && n_pv > 0) {
            wait_warp(kWsBarPV + ((n_pv - 1) & 1), par2(n_pv - 1), kT5WhereValues);
            umma::fence_after_sync();
        }
    }
    failed = __syncthreads_or(failed);
    if (where != 0) atomicOr(p.status, where);
    if ((failed || bad_page) && tid == kWsIssuer) atomicOr(p.status, failed ? kStatusWaitTimeout : kStatusBadPage);

    // ---- this range's partial result for this thread's row ----
    // (tcgen05.ld is a warp-wide instruction: every lane takes part, rows beyond the chunk only skip the stores)
    if (warp < 4) {
        const bool store = !failed && tok < p.T;
        const size_t n_vec = (size_t)p.T * Hq;
        const size_t v = (size_t)min(tok, p.T - 1) * Hq + (size_t)kvh * kGroup + head;
        float* dst = p.o_part + ((size_t)blockIdx.z * n_vec + v) * kDim;
        if (!failed && n_blk > 0) {                     // CTA-uniform
#pragma unroll
            for (int c0 = 0; c0 < kDim; c0 += 32) {
                uint32_t ov[32];
                umma::ld32(ov, tmem_o, lane0, c0);
                if (store) {
#pragma unroll
                    for (int q = 0; q < 8; ++q)
                        *reinterpret_cast<float4*>(dst + c0 + 4 * q) =
                            make_float4(__uint_as_float(ov[4 * q]), __uint_as_float(ov[4 * q + 1]),
                                        __uint_as_float(ov[4 * q + 2]), __uint_as_float(ov[4 * q + 3]));
                }
            }
        } else if (store) {
            for (int c = 0; c < kDim; c += 4) *reinterpret_cast<float4*>(dst + c) = make_float4(0.f, 0.f, 0.f, 0.f);
        }
        if (store) *reinterpret_cast<float2*>(p.ml_part + ((size_t)blockIdx.z * n_vec + v) * 2) = make_float2(m_ref, l_run);
    }
    // tensor memory goes back before the CTA exits, whatever happened above
    umma::fence_before_sync();
    __syncthreads();
    if (warp == 0) umma::tmem_free_n(tmem_base, kWsTmemCols);
}

