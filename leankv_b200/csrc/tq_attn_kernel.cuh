// Main kernel of the paged TurboQuant decode attention (included by tq_attn.cu, inside
// namespace leankv::{anonymous}; see the header comment there for the algorithm).
//
// Grid (chunk, kv head, sequence); a CTA of 4 warps covers `pages_per_cta` consecutive pages
// of one (sequence, kv head); warp w takes a contiguous quarter of them, one page (16 tokens)
// per iteration.

__device__ __forceinline__ float ex2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// Raising the running maximum rescales 32 accumulators per lane, so it is only done when a page's
// maximum exceeds the reference value by more than this many log2 units; until then probabilities
// are taken relative to the (stale) reference and stay below 2^kRescaleSlack.
constexpr float kRescaleSlack = 5.0f;

__global__ void __launch_bounds__(kAttnThreads, 6) tq_decode_attn_kernel(const AttnParams p) {
    // per-warp ring of kStages x (K chunk + V chunk); after its last page a warp reuses its ring
    // for its partial result, and the CTA reuses warp 0's ring for the merged output
    __shared__ __align__(128) uint8_t s_ring[kAttnWarps][kStages][2][kChunkBytes];
    __shared__ __align__(8) uint64_t s_bar[kAttnWarps][kStages];
    __shared__ float s_m[kAttnWarps][kGroup], s_l[kAttnWarps][kGroup];
    __shared__ int s_last;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t = lane & 3;
    const int chunk = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
    // Pull the inverse rotation (a constant, 64 KB) towards L2 early: whichever CTA ends up merging
    // the chunks needs it at the very end of the critical path.
    if (chunk == 0 && kvh == 0 && b == 0)
        for (int i = tid; i < kDim * kDim / 32; i += kAttnThreads)
            asm volatile("prefetch.global.L2 [%0];" ::"l"(p.Pi_v + i * 32));
    // Everything up to pdl_begin() may run while the launch before this one is still executing. It
    // reads only what older launches produced: the page table and every page except each sequence's
    // last one (the page the preceding append / post kernel is writing the new token into).
    const int Hq = p.H * kGroup;

    const int seq_pg0 = p.indptr[b];
    const int n_pages_b = p.indptr[b + 1] - seq_pg0;
    const int P = p.pages_per_cta;
    const int n_chunks_b = (n_pages_b + P - 1) / P;
    __half* out_base = p.out + ((size_t)b * Hq + (size_t)kvh * kGroup) * kDim;

    if (n_pages_b <= 0) {
        pdl_begin();
        if (chunk == 0)
            for (int i = tid; i < kGroup * kDim; i += kAttnThreads) out_base[i] = __float2half_rn(0.f);
        return;
    }
    if (chunk >= n_chunks_b) return;

    int last_len = p.last_len[b];
    last_len = last_len < 1 ? 1 : (last_len > 16 ? 16 : last_len);
    const int cta_pg1 = min(n_pages_b, chunk * P + P);
    const int ppw = (P + kAttnWarps - 1) / kAttnWarps;          // <= 32 (host guarantees it)
    const int w_pg0 = chunk * P + warp * ppw;
    const int n_my = max(0, min(cta_pg1, w_pg0 + ppw) - w_pg0);

    // lane i keeps the page id of this warp's i-th page; out-of-range ids are flagged once here
    int my_page = 0;
    if (lane < n_my) {
        my_page = p.indices[seq_pg0 + w_pg0 + lane];
        if (my_page < 0 || my_page >= p.n_pages) {
            my_page = -1;
            atomicOr(p.status, kStatusBadPage);
        }
    }

    const uint32_t bar0 = smem_u32(&s_bar[warp][0]);
    const uint32_t ring0 = smem_u32(&s_ring[warp][0][0][0]);
    if (lane == 0) {
#pragma unroll
        for (int s = 0; s < kStages; ++s) mbar_init(bar0 + 8 * s, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncwarp();

    const uint8_t* pool_kvh = p.pool + (size_t)kvh * kChunkBytes;
    const size_t page_stride = (size_t)2 * p.H * kChunkBytes;       // K chunk of a page -> next page
    const size_t kv_stride = (size_t)p.H * kChunkBytes;             // K chunk -> V chunk of that page
    auto issue = [&](int s, int page) {                             // lane 0 only
        const uint8_t* src = pool_kvh + (size_t)(page < 0 ? 0 : page) * page_stride;
        mbar_expect_tx(bar0 + 8 * s, 2 * kChunkBytes);
        bulk_g2s(ring0 + s * 2 * kChunkBytes, src, kChunkBytes, bar0 + 8 * s);
        bulk_g2s(ring0 + s * 2 * kChunkBytes + kChunkBytes, src + kv_stride, kChunkBytes, bar0 + 8 * s);
    };
    // first copies: all but the sequence's last page start now, that one after the wait
    const int i_seq_last = n_pages_b - 1 - w_pg0;                   // index of the last page in this warp, if it has it
#pragma unroll
    for (int s = 0; s < kStages; ++s) {
        const int pg = __shfl_sync(0xffffffffu, my_page, s);
        if (lane == 0 && s < n_my && s != i_seq_last) issue(s, pg);
    }

    pdl_begin();
    if (i_seq_last >= 0 && i_seq_last < kStages && i_seq_last < n_my) {
        const int pg = __shfl_sync(0xffffffffu, my_page, i_seq_last);
        if (lane == 0) issue(i_seq_last, pg);
    }

    // Query as the B operand of the score MMA: column n = g is (head g/2, hi|lo part g%2);
    // k-step s covers rotated coordinates 32t + 4s .. +3.
    const int head = g >> 1, part = g & 1;
    uint32_t qf[8][2];
    {
        const float* qp = p.qprime + ((size_t)b * Hq + (size_t)kvh * kGroup + head) * kDim + 32 * t;
#pragma unroll
        for (int s = 0; s < 8; ++s) {
            const float4 v = *reinterpret_cast<const float4*>(qp + 4 * s);
            qf[s][0] = pack_h2(split_part(v.x * p.qscale, part), split_part(v.y * p.qscale, part));
            qf[s][1] = pack_h2(split_part(v.z * p.qscale, part), split_part(v.w * p.qscale, part));
        }
    }

    float m_ref = -INFINITY, l_run = 0.f;     // m_ref: reference value of the exponentials (per head t)
    float acc[8][4];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;

    int n_done = 0;
    bool failed = false;
    for (int i = 0; i < n_my; ++i) {
        const int s = i & (kStages - 1);
        // the verdict is made warp-uniform so that no lane is left behind at a shuffle
        if (!__all_sync(0xffffffffu, mbar_wait_bounded(bar0 + 8 * s, (i / kStages) & 1))) {
            failed = true;
            break;
        }
        n_done = i + 1;
        const int page = __shfl_sync(0xffffffffu, my_page, i);
        const int next_page = __shfl_sync(0xffffffffu, my_page, (i + kStages) & 31);
        const int n_valid = page < 0 ? 0 : ((w_pg0 + i == n_pages_b - 1) ? last_len : 16);

        const uint8_t* stage = &s_ring[warp][s][0][0];
        const uint32_t* kw = reinterpret_cast<const uint32_t*>(stage);
        const __half* kn = reinterpret_cast<const __half*>(stage + kNormOffsetBytes);
        const uint32_t* vw = reinterpret_cast<const uint32_t*>(stage + kChunkBytes);
        const __half* vn = reinterpret_cast<const __half*>(stage + kChunkBytes + kNormOffsetBytes);

        // ---- scores: D[16 tokens][8 = 4 heads x (hi,lo)] ----
        float d[4] = {0.f, 0.f, 0.f, 0.f};
        {
            float d2[4] = {0.f, 0.f, 0.f, 0.f};   // second accumulator: halves the dependent MMA chain
            const Unit ua = load_unit(kw, lane), ub = load_unit(kw, 32 + lane);
#pragma unroll
            for (int q = 0; q < 8; ++q) {
                const uint32_t sa = ua.s[q >> 1] >> (16 * (q & 1));
                const uint32_t sb = ub.s[q >> 1] >> (16 * (q & 1));
                const uint32_t la = __byte_perm(p.tl0, p.tl1, sa), ha = __byte_perm(p.th0, p.th1, sa);
                const uint32_t lb = __byte_perm(p.tl0, p.tl1, sb), hb = __byte_perm(p.th0, p.th1, sb);
                mma_16816((q & 1) ? d2 : d, __byte_perm(la, ha, 0x5140), __byte_perm(lb, hb, 0x5140),
                          __byte_perm(la, ha, 0x7362), __byte_perm(lb, hb, 0x7362), qf[q][0], qf[q][1]);
            }
            d[0] += d2[0]; d[1] += d2[1]; d[2] += d2[2]; d[3] += d2[3];
        }
        float sa = (d[0] + d[1]) * __half2float(kn[g]);
        float sb = (d[2] + d[3]) * __half2float(kn[g + 8]);
        float na = __half2float(vn[g]), nb = __half2float(vn[g + 8]);
        if (n_valid < 16) {                      // last page of a sequence (or a rejected page)
            if (g >= n_valid) { sa = -INFINITY; na = 0.f; }
            if (g + 8 >= n_valid) { sb = -INFINITY; nb = 0.f; }
        }

        // ---- online softmax (log2 domain; the query carries scale * log2 e) ----
        float mt = fmaxf(sa, sb);
        mt = fmaxf(mt, __shfl_xor_sync(0xffffffffu, mt, 4));
        mt = fmaxf(mt, __shfl_xor_sync(0xffffffffu, mt, 8));
        mt = fmaxf(mt, __shfl_xor_sync(0xffffffffu, mt, 16));
        if (__any_sync(0xffffffffu, mt > m_ref + kRescaleSlack)) {
            if (mt > m_ref + kRescaleSlack) {         // this lane's head moves its reference value
                const float f = ex2_approx(m_ref - mt);   // 0 on the first page (m_ref = -inf)
                l_run *= f;
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    acc[j][0] *= f; acc[j][1] *= f; acc[j][2] *= f; acc[j][3] *= f;
                }
                m_ref = mt;
            }
        }
        const float m_safe = m_ref == -INFINITY ? 0.f : m_ref;    // only while nothing valid was seen
        const float pa = ex2_approx(sa - m_safe), pb = ex2_approx(sb - m_safe);
        l_run += pa + pb;
        const float wa = pa * na, wb = pb * nb;

        // Probabilities (times value norms) as the B operand of the value MMA: rows = tokens,
        // column n = g is (head g/2, hi|lo part g%2).
        const int src0 = (2 * t) * 4 + head, src1 = src0 + 4;
        const float x0 = __shfl_sync(0xffffffffu, wa, src0), x1 = __shfl_sync(0xffffffffu, wa, src1);
        const float x2 = __shfl_sync(0xffffffffu, wb, src0), x3 = __shfl_sync(0xffffffffu, wb, src1);
        // fp16 rounding of the probabilities is independent from token to token and averages out over
        // the sum, unlike rounding of the query or of the centroids: no hi/lo split here, the "lo"
        // columns of the value MMA are fed zeros
        const uint32_t b0 = part ? 0u : pack_h2(x0, x1);
        const uint32_t b1 = part ? 0u : pack_h2(x2, x3);
        {
            const Unit ua = load_unit(vw, lane), ub = load_unit(vw, 32 + lane);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const uint32_t sa2 = ua.s[j >> 1] >> (16 * (j & 1));
                const uint32_t sb2 = ub.s[j >> 1] >> (16 * (j & 1));
                const uint32_t la = __byte_perm(p.tl0, p.tl1, sa2), ha = __byte_perm(p.th0, p.th1, sa2);
                const uint32_t lb = __byte_perm(p.tl0, p.tl1, sb2), hb = __byte_perm(p.th0, p.th1, sb2);
                mma_16816(acc[j], __byte_perm(la, ha, 0x5140), __byte_perm(la, ha, 0x7362),
                          __byte_perm(lb, hb, 0x5140), __byte_perm(lb, hb, 0x7362), b0, b1);
            }
        }
        __syncwarp();   // every lane has finished reading this stage
        if (lane == 0 && i + kStages < n_my) issue(s, next_page);
    }
    if (failed) {
        // Give the copies still in flight a bounded chance to land before the CTA can exit.
        if (lane == 0) atomicOr(p.status, kStatusWaitTimeout);
        const int issued = min(n_my, n_done + kStages);
        for (int i = n_done; i < issued; ++i) mbar_wait_bounded(bar0 + 8 * (i & (kStages - 1)), (i / kStages) & 1);
    }

    // ---- warp result -> shared memory (the warp's own ring is free now) ----
    l_run += __shfl_xor_sync(0xffffffffu, l_run, 4);
    l_run += __shfl_xor_sync(0xffffffffu, l_run, 8);
    l_run += __shfl_xor_sync(0xffffffffu, l_run, 16);
    if (g == 0) {
        s_m[warp][t] = m_ref;
        s_l[warp][t] = l_run;
    }
    __syncwarp();
    float* w_acc = reinterpret_cast<float*>(&s_ring[warp][0][0][0]);      // [kGroup][kDim] floats = 2 KB
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        // rows g / g+8 of m-tile j are rotated coordinates 16g+2j / 16g+2j+1; columns 2t, 2t+1
        // are the hi and lo parts of head t.
        *reinterpret_cast<float2*>(&w_acc[t * kDim + 16 * g + 2 * j]) =
            make_float2(acc[j][0] + acc[j][1], acc[j][2] + acc[j][3]);
    }
    __syncthreads();

    // ---- CTA merge over its 4 warps: thread = rotated coordinate ----
    float* ring_f = reinterpret_cast<float*>(&s_ring[0][0][0][0]);
    constexpr int kWarpRingFloats = kStages * 2 * kChunkBytes / 4;
    float o[kGroup], mh[kGroup], lh[kGroup];
#pragma unroll
    for (int h = 0; h < kGroup; ++h) {
        float m = s_m[0][h];
#pragma unroll
        for (int w = 1; w < kAttnWarps; ++w) m = fmaxf(m, s_m[w][h]);
        float ov = 0.f, lv = 0.f;
#pragma unroll
        for (int w = 0; w < kAttnWarps; ++w) {
            const float mw = s_m[w][h];
            const float f = mw == -INFINITY ? 0.f : ex2_approx(mw - m);
            ov = fmaf(f, ring_f[w * kWarpRingFloats + h * kDim + tid], ov);
            lv = fmaf(f, s_l[w][h], lv);
        }
        o[h] = ov; mh[h] = m; lh[h] = lv;
    }

    if (n_chunks_b > 1) {
        float* mine = p.partials + (((size_t)b * p.H + kvh) * p.n_chunks + chunk) * kPartialFloats;
#pragma unroll
        for (int h = 0; h < kGroup; ++h) mine[h * kDim + tid] = o[h];
        if (tid < kGroup) {
            mine[kGroup * kDim + tid] = mh[tid];
            mine[kGroup * kDim + kGroup + tid] = lh[tid];
        }
        __threadfence();
        __syncthreads();
        if (tid == 0) {
            const int prev = atomicAdd(&p.counters[b * p.H + kvh], 1);
            s_last = (prev == n_chunks_b - 1);
        }
        __syncthreads();
        if (!s_last) return;
        __threadfence();
        // last CTA of this (sequence, kv head): merge the chunk partials in chunk order.
        // All maxima / sums first (one round trip, staged in the now idle ring), then the value rows
        // with the loads of several chunks and all four heads in flight together.
        const float* base = p.partials + (((size_t)b * p.H + kvh) * p.n_chunks) * kPartialFloats;
        float* s_ml = ring_f;                                     // [n_chunks_b][2 * kGroup]: m then l
        for (int i = tid; i < n_chunks_b * 2 * kGroup; i += kAttnThreads)
            s_ml[i] = ld_cg_f32(base + (size_t)(i >> 3) * kPartialFloats + kGroup * kDim + (i & 7));
        __syncthreads();
        float mg[kGroup];
#pragma unroll
        for (int h = 0; h < kGroup; ++h) {
            float m = -INFINITY;
            for (int c = 0; c < n_chunks_b; ++c) m = fmaxf(m, s_ml[c * 2 * kGroup + h]);
            mg[h] = m;
            o[h] = 0.f;
            lh[h] = 0.f;
        }
#pragma unroll 4
        for (int c = 0; c < n_chunks_b; ++c) {
            const float* pc = base + (size_t)c * kPartialFloats + tid;
            float ov[kGroup];
#pragma unroll
            for (int h = 0; h < kGroup; ++h) ov[h] = ld_cg_f32(pc + h * kDim);
#pragma unroll
            for (int h = 0; h < kGroup; ++h) {
                const float mc = s_ml[c * 2 * kGroup + h];
                const float f = mc == -INFINITY ? 0.f : ex2_approx(mc - mg[h]);
                o[h] = fmaf(f, ov[h], o[h]);
                lh[h] = fmaf(f, s_ml[c * 2 * kGroup + kGroup + h], lh[h]);
            }
        }
        __syncthreads();                                          // s_ml is overwritten below (s_o / s_part)
        if (tid == 0) p.counters[b * p.H + kvh] = 0;
    }

    // ---- normalise, undo the centroid scale, rotate back: out = o @ Pi_v ----
    float* s_o = ring_f + 512;               // [kGroup][kDim], behind warp 0's partial
    float* s_part = ring_f + 1024;           // [kAttnWarps][kGroup][kDim]
#pragma unroll
    for (int h = 0; h < kGroup; ++h) s_o[h * kDim + tid] = lh[h] > 0.f ? o[h] * (p.inv_alpha / lh[h]) : 0.f;
    __syncthreads();
    {
        // warp w sums rows 32w .. 32w+31 of Pi_v for 4 output columns per lane (coalesced 16-byte loads)
        float r[kGroup][4];
#pragma unroll
        for (int h = 0; h < kGroup; ++h) r[h][0] = r[h][1] = r[h][2] = r[h][3] = 0.f;
        const float4* pv = reinterpret_cast<const float4*>(p.Pi_v) + (size_t)(32 * warp) * (kDim / 4) + lane;
#pragma unroll
        for (int ii = 0; ii < 32; ++ii) {
            const float4 w4 = __ldg(pv + (size_t)ii * (kDim / 4));
            const int i = 32 * warp + ii;
#pragma unroll
            for (int h = 0; h < kGroup; ++h) {
                const float sv = s_o[h * kDim + i];
                r[h][0] = fmaf(sv, w4.x, r[h][0]);
                r[h][1] = fmaf(sv, w4.y, r[h][1]);
                r[h][2] = fmaf(sv, w4.z, r[h][2]);
                r[h][3] = fmaf(sv, w4.w, r[h][3]);
            }
        }
#pragma unroll
        for (int h = 0; h < kGroup; ++h)
            *reinterpret_cast<float4*>(&s_part[(warp * kGroup + h) * kDim + 4 * lane]) =
                make_float4(r[h][0], r[h][1], r[h][2], r[h][3]);
    }
    __syncthreads();
#pragma unroll
    for (int h = 0; h < kGroup; ++h) {
        float v = 0.f;
#pragma unroll
        for (int w = 0; w < kAttnWarps; ++w) v += s_part[(w * kGroup + h) * kDim + tid];
        out_base[h * kDim + tid] = __float2half_rn(v);
    }
}
