// Main kernel of the paged TurboQuant decode attention (included by tq_attn.cu, inside
// namespace leankv::{anonymous}; see the header comment there for the algorithm).
//
// Work split. All pages of all (sequence, kv head) pairs form one flat list, ordered by sequence,
// then kv head, then page. The grid is one wave of resident CTAs and CTA c takes the c-th equal
// share of that list (shares differ by at most one page), whatever the sequence lengths are. A
// share is cut at pair boundaries into segments; the CTA's four warps split each segment's pages,
// their results are merged in shared memory, and a segment that is not a whole pair leaves a
// partial result in the workspace. The last CTA to arrive for a pair merges the partials in CTA
// order and applies the inverse value rotation. When there are at least as many CTAs as pairs the
// CTA count is rounded down to a multiple of the pair count, so that for sequences of equal length
// (a single sequence in particular) no share crosses a pair boundary.

__device__ __forceinline__ float ex2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// Raising the running maximum rescales 32 accumulators per lane, so it is only done when a page's
// maximum exceeds the reference value by more than this many log2 units; until then probabilities
// are taken relative to the (stale) reference and stay below 2^kRescaleSlack.
constexpr float kRescaleSlack = 5.0f;
// Reference value before any valid token has been seen: finite, so that no special case is needed
// (any real score exceeds it by more than the slack, and 2^(kNoRef - m) is 0).
constexpr float kNoRef = -1.0e30f;

// Integer MMA accumulators start from the bit pattern of 1.5 * 2^23: adding an integer |n| < 2^22 to
// that pattern gives the bit pattern of the float 1.5 * 2^23 + n, so the sums come out of the tensor
// core as floats without a conversion instruction.
constexpr float kBiasF = 12582912.0f;

// kClusterCtas > 0: the CTAs of a (sequence, kv head) pair form one thread-block cluster of that many CTAs
// (see the end of the kernel); used when a cluster per pair fits into one wave. 0: the general kernel.
template <int kOcc, int kClusterCtas>   // kOcc: resident CTAs per SM the register allocation is held to
__global__ void __launch_bounds__(kAttnThreads, kOcc) tq_decode_attn_kernel(const AttnParams p) {
    constexpr bool kCluster = kClusterCtas > 0;
    // per-warp ring of kStages x (K chunk + V chunk)
    __shared__ __align__(128) uint8_t s_ring[kAttnWarps][kStages][2][kChunkBytes];
    __shared__ __align__(8) uint64_t s_bar[kAttnWarps][kStages];
    __shared__ __align__(16) float s_res[kAttnWarps][kGroup][kDim];   // warp results, later scratch of the merge
    __shared__ float s_m[kAttnWarps][kGroup], s_l[kAttnWarps][kGroup];
    __shared__ int s_ip[kAttnThreads];                                // kv_indptr of a small batch
    __shared__ int s_last;
    static_assert(kStages == 4, "the page loop is unrolled over a 4-slot ring");

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t = lane & 3;
    const int H = p.H, Hq = H * kGroup;
    // The eight look-up table words are used by ~100 byte permutes per page: hold them in registers
    // (an opaque move keeps the compiler from re-reading the parameter bank at every use).
    uint32_t kh0, kh1, kl0, kl1, tl0, tl1, th0, th1;
    asm volatile("mov.b32 %0, %1;" : "=r"(kh0) : "r"(p.kh0));
    asm volatile("mov.b32 %0, %1;" : "=r"(kh1) : "r"(p.kh1));
    asm volatile("mov.b32 %0, %1;" : "=r"(kl0) : "r"(p.kl0));
    asm volatile("mov.b32 %0, %1;" : "=r"(kl1) : "r"(p.kl1));
    asm volatile("mov.b32 %0, %1;" : "=r"(tl0) : "r"(p.tl0));
    asm volatile("mov.b32 %0, %1;" : "=r"(tl1) : "r"(p.tl1));
    asm volatile("mov.b32 %0, %1;" : "=r"(th0) : "r"(p.th0));
    asm volatile("mov.b32 %0, %1;" : "=r"(th1) : "r"(p.th1));
    bool waited = (p.flags & LEANKV_ATTN_EARLY_FETCH) == 0;
    if (waited) pdl_begin();
    // Pull the inverse rotation (a constant, 64 KB) towards L2 early: whichever CTA ends up merging
    // needs it at the very end of the critical path.
    if (blockIdx.x == 0)
        for (int i = tid; i < kDim * kDim / 32; i += kAttnThreads)
            asm volatile("prefetch.global.L2 [%0];" ::"l"(p.Pi_v + i * 32));

    const uint32_t bar0 = smem_u32(&s_bar[warp][0]);
    const uint32_t ring0 = smem_u32(&s_ring[warp][0][0][0]);
    if (lane == 0) {
#pragma unroll
        for (int s = 0; s < kStages; ++s) mbar_init(bar0 + 8 * s, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncwarp();

    // ---- this CTA's share of the flat page list ----
    // With early fetch everything up to the first pdl_begin() below runs while the launch before this
    // one may still be executing; it reads only the page table and pages that older launches wrote.
    // A batch of fewer than 128 sequences has its whole indptr fetched in one go (one memory round trip
    // before the page ids can be asked for); larger batches read it from global memory as needed.
    const bool small_b = p.B < kAttnThreads;
    if (small_b) {
        if (tid <= p.B) s_ip[tid] = p.indptr[tid];
        __syncthreads();
    }
    auto ip = [&](int i) -> int { return small_b ? s_ip[i] : p.indptr[i]; };
    const int ip0 = ip(0);
    long long F = 0, C = 1, f_lo = 0, f_hi = 0;
    bool fits32 = true;
    int b = 0, seq_pg0 = 0, n_b = 0, kvh = 0, pg = 0;
    // floor(c * F / C) and its inverse; 32-bit arithmetic when the products fit (the usual case)
    auto share_start = [&](long long c) -> long long {
        return fits32 ? (long long)((unsigned)c * (unsigned)F / (unsigned)C) : c * F / C;
    };
    auto cta_of = [&](long long f) -> int {        // the CTA whose share holds flat page f
        return fits32 ? (int)(((unsigned)(f + 1) * (unsigned)C + (unsigned)F - 1u) / (unsigned)F) - 1
                      : (int)(((f + 1) * C + F - 1) / F) - 1;
    };
    unsigned crank = 0;                   // this CTA's rank in its cluster
    if constexpr (kCluster) {
        // cluster = pair; rank r takes pages [r n / kClusterCtas, (r + 1) n / kClusterCtas) of the pair's n
        asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(crank));
        const int pair = blockIdx.x / kClusterCtas;
        b = pair / H;
        kvh = pair - b * H;
        seq_pg0 = ip(b);
        n_b = max(ip(b + 1) - seq_pg0, 0);
        pg = (int)((unsigned)n_b * crank / kClusterCtas);
        f_hi = (int)((unsigned)n_b * (crank + 1) / kClusterCtas) - pg;     // the loop below runs over [0, f_hi)
    } else {
    F = (long long)H * (ip(p.B) - ip0);
    // sequences without pages produce zeros; CTAs share them out
    for (int bz = blockIdx.x; bz < p.B; bz += gridDim.x) {
        if (ip(bz + 1) - ip(bz) <= 0) {
            if (!waited) { pdl_begin(); waited = true; }
            __half* o = p.out + (size_t)bz * Hq * kDim;
            for (int i = tid; i < Hq * kDim; i += kAttnThreads) o[i] = __float2half_rn(0.f);
        }
    }
    C = gridDim.x;
    {
        // no more CTAs than give each about kMinPagesPerCta pages; whole multiples of the pair count, so that
        // equal-length sequences are cut into equal pieces that end at pair boundaries
        const long long pairs = (long long)p.B * H;
        long long cap = (F + kMinPagesPerCta - 1) / kMinPagesPerCta;
        if (cap >= pairs) cap = (cap + pairs - 1) / pairs * pairs;
        if (cap < 1) cap = 1;
        if (C > cap) C = cap;
        if (C >= pairs) C -= C % pairs;
    }
    if (F <= 0 || (long long)blockIdx.x >= C) {
        if (!waited) pdl_begin();
        return;
    }
    fits32 = (F + 1) * C + F < (1ll << 32);
    f_lo = share_start(blockIdx.x);
    f_hi = share_start((long long)blockIdx.x + 1);

    // sequence that holds flat page f_lo: the last b with H * (indptr[b] - indptr[0]) <= f_lo
    {
        int lo = 0, hi = p.B;
        while (hi - lo > 1) {
            const int step = (hi - lo + kAttnThreads - 1) / kAttnThreads;
            const long long idx = (long long)lo + (long long)(tid + 1) * step;
            const bool pred = idx < hi && (long long)H * (ip((int)idx) - ip0) <= f_lo;
            const int cnt = __syncthreads_count(pred);
            lo += cnt * step;
            hi = min(hi, lo + step);
        }
        b = lo;
    }
    seq_pg0 = ip(b);
    n_b = ip(b + 1) - seq_pg0;
    {
        const long long r = f_lo - (long long)H * (seq_pg0 - ip0);    // < H * n_b
        kvh = fits32 ? (int)((unsigned)r / (unsigned)n_b) : (int)(r / n_b);
        pg = (int)(r - (long long)kvh * n_b);
    }
    }

    const size_t page_stride = (size_t)2 * H * kChunkBytes;       // K chunk of a page -> next page
    const size_t kv_stride = (size_t)H * kChunkBytes;             // K chunk -> V chunk of that page
    const int l4 = lane & 3;
    unsigned phase = 0;              // bit s: parity the next wait on ring slot s looks for
    unsigned inflight = 0;           // bit s: a copy into ring slot s has been issued and not yet waited for
    bool failed = false;             // a bounded wait gave up: the warp stops using its ring
    bool have_partial = false;       // cluster mode: the loop below left this CTA's partial result in shared memory

    for (long long f = f_lo; f < f_hi;) {
        const int seg_len = (int)min((long long)(n_b - pg), f_hi - f);
        if (seg_len <= 0) break;         // cannot happen for a consistent page table; never loop on an inconsistent one
        const bool whole = !kCluster && seg_len == n_b;
        // ---- this warp's pages of the segment ----
        const int w_lo = pg + (int)(((long long)seg_len * warp) / kAttnWarps);
        const int w_hi = pg + (int)(((long long)seg_len * (warp + 1)) / kAttnWarps);
        const int n_my = failed ? 0 : w_hi - w_lo;
        const uint8_t* pool_kvh = p.pool + (size_t)kvh * kChunkBytes;
        // lane s (s < 4) feeds ring slot s
        auto issue = [&](int page) {
            const uint8_t* src = pool_kvh + (size_t)(page < 0 ? 0 : page) * page_stride;
            const uint32_t bar = bar0 + 8 * l4, dst = ring0 + l4 * 2 * kChunkBytes;
            mbar_expect_tx(bar, 2 * kChunkBytes);
            bulk_g2s(dst, src, kChunkBytes, bar);
            bulk_g2s(dst + kChunkBytes, src + kv_stride, kChunkBytes, bar);
        };
        // Page ids travel in groups of four: lane (any g, l4) holds the id of page base + l4 (lanes with
        // equal l4 read the same word). Ids outside the pool are flagged once and read as pages without
        // valid tokens.
        auto fetch = [&](int base) -> int {
            int id = 0;
            if (base + l4 < n_my) {
                id = p.indices[seq_pg0 + w_lo + base + l4];
                if (id < 0 || id >= p.n_pages) {
                    id = -1;
                    if (lane < 4) atomicOr(p.status, kStatusBadPage);
                }
            }
            return id;
        };
        int id_cur = fetch(0), id_nxt = fetch(kStages);
        // first copies; before the dependency wait the sequence's last page (the one the preceding
        // launch may be writing the new token into) is left out and issued right after the wait
        {
            const int i_seq_last = n_b - 1 - w_lo;
            const bool mine0 = lane < kStages && lane < n_my;
            const bool hold = !waited && lane == i_seq_last;
            if (mine0 && !hold) issue(id_cur);
            if (!waited) {
                pdl_begin();
                waited = true;
                if (mine0 && hold) issue(id_cur);
            }
            inflight |= (1u << min(n_my, kStages)) - 1u;
        }

        // ---- query as the A operand of the integer score MMA ----
        // One m16n8k32 step covers 32 coordinates: rows 0..7 hold the high digit of the query, rows 8..15
        // its low digit (heads 0..3, repeated in rows 4..7 so that all lanes do the same work). Multiplied
        // with the centroids' high digits that gives HH (rows 0..7) and q_lo x c_hi (rows 8..15); with the
        // centroids' low digits q_hi x c_lo and q_lo x c_lo. Lane (g, t) holds head g & 3, rotated
        // coordinates 32t .. 32t+31; k-block kb covers coordinates 32t + 8kb .. +7.
        uint32_t qa[4][4];
        float kscale;            // score per integer unit of (256 * HH + MID), before the key norm
        {
            const int head = g & 3;
            const float* qp = p.qprime + ((size_t)b * Hq + (size_t)kvh * kGroup + head) * kDim + 32 * t;
            float4 v[8];
            float amax = 0.f;
#pragma unroll
            for (int s = 0; s < 8; ++s) {
                v[s] = *reinterpret_cast<const float4*>(qp + 4 * s);
                amax = fmaxf(amax, fmaxf(fmaxf(fabsf(v[s].x), fabsf(v[s].y)), fmaxf(fabsf(v[s].z), fabsf(v[s].w))));
            }
            amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
            amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
            const float uq = amax > 0.f ? amax * (1.0f / kFixedMax) : 1.0f;
            const float inv = 1.0f / uq;
            kscale = 256.0f * uq * p.c_unit * p.qscale;
            auto digits = [&](float x, int sh, uint32_t& hi, uint32_t& lo) {
                const int qi = __float2int_rn(x * inv);
                const int h8 = (qi + 128) >> 8;                       // |qi| <= 32512 keeps this in [-127, 127]
                const int l8 = qi - (h8 << 8);                        // balanced low digit in [-128, 127]
                hi |= (uint32_t)(h8 & 255) << sh;
                lo |= (uint32_t)(l8 & 255) << sh;
            };
#pragma unroll
            for (int s = 0; s < 8; ++s) {
                uint32_t hi = 0, lo = 0;
                digits(v[s].x, 0, hi, lo);
                digits(v[s].y, 8, hi, lo);
                digits(v[s].z, 16, hi, lo);
                digits(v[s].w, 24, hi, lo);
                qa[s >> 1][2 * (s & 1)] = hi;          // a0 / a2: rows 0..7, k 0..15 / 16..31
                qa[s >> 1][2 * (s & 1) + 1] = lo;      // a1 / a3: rows 8..15
            }
        }

        float m_ref = kNoRef, l_run = 0.f;        // head g & 3, this lane's four tokens per page
        float acc[8][4];
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;
        const int last_len = min(max(p.last_len[b], 1), 16);

        // One page; n_valid < 16 for a sequence's last page and 0 for a page id that was rejected. The body
        // exists once (it is a few hundred instructions: copies of it would not fit the instruction cache
        // close to the schedulers).
        auto do_page = [&](const uint8_t* stage, int n_valid) {
            const uint32_t* kw = reinterpret_cast<const uint32_t*>(stage);
            const uint32_t* kn2 = reinterpret_cast<const uint32_t*>(stage + kNormOffsetBytes);
            const uint32_t* vw = reinterpret_cast<const uint32_t*>(stage + kChunkBytes);
            const uint32_t* vn2 = reinterpret_cast<const uint32_t*>(stage + kChunkBytes + kNormOffsetBytes);

            // ---- scores: D[row][token], tokens 0..7 in tile 0 and 8..15 in tile 1 ----
            int dh0[4], dl0[4], dh1[4], dl1[4];       // centroid high / low digits, tile 0 / 1
            {
                const Unit ua = load_unit(kw, lane), ub = load_unit(kw, 32 + lane);
#pragma unroll
                for (int kb = 0; kb < 4; ++kb) {
                    const uint32_t sa = ua.s[kb], sa2 = sa >> 16, sb = ub.s[kb], sb2 = sb >> 16;
                    const uint32_t ah0 = __byte_perm(kh0, kh1, sa), ah1 = __byte_perm(kh0, kh1, sa2);
                    const uint32_t al0 = __byte_perm(kl0, kl1, sa), al1 = __byte_perm(kl0, kl1, sa2);
                    const uint32_t bh0 = __byte_perm(kh0, kh1, sb), bh1 = __byte_perm(kh0, kh1, sb2);
                    const uint32_t bl0 = __byte_perm(kl0, kl1, sb), bl1 = __byte_perm(kl0, kl1, sb2);
                    if (kb == 0) {
                        mma_s8_16832_bias(dh0, qa[kb], ah0, ah1);
                        mma_s8_16832_bias(dl0, qa[kb], al0, al1);
                        mma_s8_16832_bias(dh1, qa[kb], bh0, bh1);
                        mma_s8_16832_bias(dl1, qa[kb], bl0, bl1);
                    } else {
                        mma_s8_16832(dh0, qa[kb], ah0, ah1);
                        mma_s8_16832(dl0, qa[kb], al0, al1);
                        mma_s8_16832(dh1, qa[kb], bh0, bh1);
                        mma_s8_16832(dl1, qa[kb], bl0, bl1);
                    }
                }
            }
            // tokens of this lane: 2t, 2t+1 (tile 0) and 8+2t, 9+2t (tile 1); norms as fp16 pairs
            const float2 kna = h2_to_f2(kn2[t]), knb = h2_to_f2(kn2[4 + t]);
            float2 vna = h2_to_f2(vn2[t]), vnb = h2_to_f2(vn2[4 + t]);
            // 256 * HH + (q_lo c_hi + q_hi c_lo): c0/c1 of the high-digit tile are HH, its c2/c3 and the
            // low-digit tile's c0/c1 are the two mixed sums. Every sum carries the accumulator bias; all
            // three subtractions are exact.
            auto val = [](const int (&dh)[4], const int (&dl)[4], int c) -> float {
                const float mid = (__int_as_float(dh[2 + c]) - 2.f * kBiasF) + __int_as_float(dl[c]);
                return fmaf(__int_as_float(dh[c]) - kBiasF, 256.f, mid);
            };
            const float v0 = val(dh0, dl0, 0), v1 = val(dh0, dl0, 1), v2 = val(dh1, dl1, 0), v3 = val(dh1, dl1, 1);
            const float k0 = kscale * kna.x, k1 = kscale * kna.y, k2 = kscale * knb.x, k3 = kscale * knb.y;
            // scores relative to the reference value (log2 domain; the scale carries log2 e)
            float s0 = fmaf(v0, k0, -m_ref), s1 = fmaf(v1, k1, -m_ref), s2 = fmaf(v2, k2, -m_ref),
                  s3 = fmaf(v3, k3, -m_ref);
            // tokens beyond n_valid are masked out
            const bool x0 = 2 * t >= n_valid, x1 = 2 * t + 1 >= n_valid, x2 = 8 + 2 * t >= n_valid, x3 = 9 + 2 * t >= n_valid;
            if (x0) { s0 = -INFINITY; vna.x = 0.f; }
            if (x1) { s1 = -INFINITY; vna.y = 0.f; }
            if (x2) { s2 = -INFINITY; vnb.x = 0.f; }
            if (x3) { s3 = -INFINITY; vnb.y = 0.f; }
            // ---- online softmax ----
            const float mx = fmaxf(fmaxf(s0, s1), fmaxf(s2, s3));
            if (__any_sync(0xffffffffu, mx > kRescaleSlack)) {
                // some head's reference value moves: its lanes agree on the page's true maximum as the new
                // one, and every lane rescales the accumulator columns of the heads it holds
                float mh = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
                mh = fmaxf(mh, __shfl_xor_sync(0xffffffffu, mh, 2));
                const float r0 = x0 ? -INFINITY : v0 * k0, r1 = x1 ? -INFINITY : v1 * k1;
                const float r2 = x2 ? -INFINITY : v2 * k2, r3 = x3 ? -INFINITY : v3 * k3;
                float tm = fmaxf(fmaxf(r0, r1), fmaxf(r2, r3));
                tm = fmaxf(tm, __shfl_xor_sync(0xffffffffu, tm, 1));
                tm = fmaxf(tm, __shfl_xor_sync(0xffffffffu, tm, 2));
                float fsc = 1.0f;
                if (mh > kRescaleSlack) {
                    fsc = ex2_approx(m_ref - tm);          // 0 on the first page (m_ref = kNoRef)
                    l_run *= fsc;
                    m_ref = tm;
                    s0 = r0 - tm; s1 = r1 - tm; s2 = r2 - tm; s3 = r3 - tm;
                }
                const float fa = __shfl_sync(0xffffffffu, fsc, ((2 * t) & 3) * 4);
                const float fb = __shfl_sync(0xffffffffu, fsc, ((2 * t + 1) & 3) * 4);
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    acc[j][0] *= fa; acc[j][2] *= fa;
                    acc[j][1] *= fb; acc[j][3] *= fb;
                }
            }
            const float p0 = ex2_approx(s0), p1 = ex2_approx(s1), p2 = ex2_approx(s2), p3 = ex2_approx(s3);
            l_run += (p0 + p1) + (p2 + p3);
            // Probabilities (times value norms) are already where the value MMA wants its B operand:
            // rows = tokens 2t, 2t+1, 2t+8, 2t+9, column g = head g & 3 (columns 4..7 repeat 0..3 and are
            // never stored). fp16 rounding of the probabilities is independent from token to token and
            // averages out over the sum.
            const uint32_t b0 = pack_h2(p0 * vna.x, p1 * vna.y);
            const uint32_t b1 = pack_h2(p2 * vnb.x, p3 * vnb.y);
            {
                const Unit ua = load_unit(vw, lane), ub = load_unit(vw, 32 + lane);
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const uint32_t sa2 = ua.s[j >> 1] >> (16 * (j & 1));
                    const uint32_t sb2 = ub.s[j >> 1] >> (16 * (j & 1));
                    const uint32_t la = __byte_perm(tl0, tl1, sa2), ha = __byte_perm(th0, th1, sa2);
                    const uint32_t lb = __byte_perm(tl0, tl1, sb2), hb = __byte_perm(th0, th1, sb2);
                    mma_16816(acc[j], __byte_perm(la, ha, 0x5140), __byte_perm(la, ha, 0x7362),
                              __byte_perm(lb, hb, 0x5140), __byte_perm(lb, hb, 0x7362), b0, b1);
                }
            }
        };

        int id_nn = fetch(2 * kStages);                      // two groups ahead, in flight while a group is processed
        unsigned bad = __ballot_sync(0xffffffffu, id_cur < 0) & 0xFu;
        for (int i = 0; i < n_my; ++i) {
            const int s = i & (kStages - 1);
            const uint32_t bar = bar0 + 8 * s;
            // the verdict is made warp-uniform so that no lane is left behind at a shuffle
            if (!__all_sync(0xffffffffu, mbar_wait_bounded(bar, (phase >> s) & 1u))) {
                failed = true;
                break;
            }
            phase ^= 1u << s;
            inflight &= ~(1u << s);
            const int n_valid = ((bad >> s) & 1u) ? 0 : (w_lo + i == n_b - 1 ? last_len : 16);
            do_page(&s_ring[warp][0][0][0] + s * (2 * kChunkBytes), n_valid);
            __syncwarp();   // every lane has finished reading this slot
            if (i + kStages < n_my) {
                if (lane == s) issue(id_nxt);
                inflight |= 1u << s;
            }
            if (s == kStages - 1) {                          // next group
                id_cur = id_nxt;
                id_nxt = id_nn;
                id_nn = fetch(i + 1 + 2 * kStages);
                bad = __ballot_sync(0xffffffffu, id_cur < 0) & 0xFu;
            }
        }
        if (failed && inflight != 0) {
            // Give the copies still in flight a bounded chance to land before the CTA can exit.
            if (lane == 0) atomicOr(p.status, kStatusWaitTimeout);
#pragma unroll
            for (int s = 0; s < kStages; ++s)
                if ((inflight >> s) & 1u) mbar_wait_bounded(bar0 + 8 * s, (phase >> s) & 1u);
            inflight = 0;
        }

        // ---- warp result -> shared memory ----
        l_run += __shfl_xor_sync(0xffffffffu, l_run, 1);
        l_run += __shfl_xor_sync(0xffffffffu, l_run, 2);
        if (g < 4 && t == 0) {                     // lanes g >= 4 hold copies of heads 0..3
            s_m[warp][g] = m_ref;
            s_l[warp][g] = l_run;
        }
        if (t < 2) {
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                // rows g / g+8 of m-tile j are rotated coordinates 16g+2j / 16g+2j+1; columns 2t, 2t+1
                // are heads 2t and 2t+1.
                *reinterpret_cast<float2*>(&s_res[warp][2 * t][16 * g + 2 * j]) = make_float2(acc[j][0], acc[j][2]);
                *reinterpret_cast<float2*>(&s_res[warp][2 * t + 1][16 * g + 2 * j]) = make_float2(acc[j][1], acc[j][3]);
            }
        }
        __syncthreads();

        // ---- CTA merge over its 4 warps: thread = rotated coordinate ----
        float o[kGroup], mh[kGroup], lh[kGroup];
#pragma unroll
        for (int h = 0; h < kGroup; ++h) {
            float m = s_m[0][h];
#pragma unroll
            for (int w = 1; w < kAttnWarps; ++w) m = fmaxf(m, s_m[w][h]);
            float ov = 0.f, lv = 0.f;
#pragma unroll
            for (int w = 0; w < kAttnWarps; ++w) {
                const float fw = ex2_approx(s_m[w][h] - m);
                ov = fmaf(fw, s_res[w][h][tid], ov);
                lv = fmaf(fw, s_l[w][h], lv);
            }
            o[h] = ov; mh[h] = m; lh[h] = lv;
        }
        __syncthreads();                       // s_res / s_m / s_l may be overwritten from here on

        if constexpr (kCluster) {
            // this CTA's partial result stays in its shared memory for the other CTAs of the cluster
#pragma unroll
            for (int h = 0; h < kGroup; ++h) s_res[0][h][tid] = o[h];
            if (tid < kGroup) {
                s_m[0][tid] = mh[tid];
                s_l[0][tid] = lh[tid];
            }
            have_partial = true;
            break;
        }

        bool finish = whole;
        if (!whole) {
            // partial slot: 1 if this pair started in an earlier part of this CTA's share (it is then
            // the CTA's last segment), 0 if the CTA's share starts inside or at the start of the pair
            const long long o_p = (long long)H * (seq_pg0 - ip0) + (long long)kvh * n_b;
            const int slot = f_lo < o_p ? 1 : 0;
            float* mine = p.partials + ((size_t)blockIdx.x * 2 + slot) * kPartialFloats;
#pragma unroll
            for (int h = 0; h < kGroup; ++h) mine[h * kDim + tid] = o[h];
            if (tid < kGroup) {
                mine[kGroup * kDim + tid] = mh[tid];
                mine[kGroup * kDim + kGroup + tid] = lh[tid];
            }
            __threadfence();
            __syncthreads();
            const int c_first = cta_of(o_p), c_last = cta_of(o_p + n_b - 1);
            const int n_seg = c_last - c_first + 1;
            if (tid == 0) {
                const int prev = atomicAdd(&p.counters[b * H + kvh], 1);
                __threadfence();               // the other CTAs' partials are read after this point
                s_last = (prev == n_seg - 1);
            }
            __syncthreads();
            if (s_last) {
                // last CTA of this (sequence, kv head): merge the partials in CTA order. Maxima / sums and the
                // value rows of the first pieces travel in the same round trip.
                float* s_ml = &s_res[0][0][0];                            // [n_seg][2 * kGroup]: m then l
                const int first_slot = share_start(c_first) < o_p ? 1 : 0;
                auto part_of = [&](int k) -> const float* {
                    return p.partials + ((size_t)(c_first + k) * 2 + (k == 0 ? first_slot : 0)) * kPartialFloats;
                };
                // a pair cut into more pieces than the staging area holds (one very long sequence among
                // short ones) reads its maxima / sums from the workspace directly
                const bool staged = n_seg * 2 * kGroup <= kAttnWarps * kGroup * kDim;
                auto ml = [&](int k, int j) -> float {
                    return staged ? s_ml[k * 2 * kGroup + j] : ld_cg_f32(part_of(k) + kGroup * kDim + j);
                };
                if (staged)
                    for (int i = tid; i < n_seg * 2 * kGroup; i += kAttnThreads)
                        s_ml[i] = ld_cg_f32(part_of(i >> 3) + kGroup * kDim + (i & 7));
                constexpr int kMergeBatch = 12;
                float ov0[kMergeBatch][kGroup];
#pragma unroll
                for (int k = 0; k < kMergeBatch; ++k) {
                    const float* pc = part_of(k < n_seg ? k : 0) + tid;
#pragma unroll
                    for (int h = 0; h < kGroup; ++h) ov0[k][h] = k < n_seg ? ld_cg_f32(pc + h * kDim) : 0.f;
                }
                __syncthreads();
                float mg[kGroup];
#pragma unroll
                for (int h = 0; h < kGroup; ++h) {
                    float m = kNoRef;
                    for (int k = 0; k < n_seg; ++k) m = fmaxf(m, ml(k, h));
                    mg[h] = m;
                    o[h] = 0.f;
                    lh[h] = 0.f;
                }
#pragma unroll
                for (int k = 0; k < kMergeBatch; ++k) {
                    if (k < n_seg) {
#pragma unroll
                        for (int h = 0; h < kGroup; ++h) {
                            const float fc = ex2_approx(ml(k, h) - mg[h]);
                            o[h] = fmaf(fc, ov0[k][h], o[h]);
                            lh[h] = fmaf(fc, ml(k, kGroup + h), lh[h]);
                        }
                    }
                }
#pragma unroll 4
                for (int k = kMergeBatch; k < n_seg; ++k) {
                    const float* pc = part_of(k) + tid;
                    float ov[kGroup];
#pragma unroll
                    for (int h = 0; h < kGroup; ++h) ov[h] = ld_cg_f32(pc + h * kDim);
#pragma unroll
                    for (int h = 0; h < kGroup; ++h) {
                        const float fc = ex2_approx(ml(k, h) - mg[h]);
                        o[h] = fmaf(fc, ov[h], o[h]);
                        lh[h] = fmaf(fc, ml(k, kGroup + h), lh[h]);
                    }
                }
                __syncthreads();                                          // s_ml is overwritten below
                if (tid == 0) p.counters[b * H + kvh] = 0;
                finish = true;
            }
        }

        if (finish) {
            // ---- normalise, undo the centroid scale, rotate back: out = o @ Pi_v ----
            float* s_o = &s_res[0][0][0];                                 // [kGroup][kDim]
            float* s_part = &s_res[1][0][0];                              // [kAttnWarps - 1][kGroup][kDim]
#pragma unroll
            for (int h = 0; h < kGroup; ++h) s_o[h * kDim + tid] = lh[h] > 0.f ? o[h] * (p.inv_alpha / lh[h]) : 0.f;
            __syncthreads();
            // warp w sums rows 32w .. 32w+31 of Pi_v for 4 output columns per lane (coalesced 16-byte loads)
            float r[kGroup][4];
#pragma unroll
            for (int h = 0; h < kGroup; ++h) r[h][0] = r[h][1] = r[h][2] = r[h][3] = 0.f;
            const float4* pv = reinterpret_cast<const float4*>(p.Pi_v) + (size_t)(32 * warp) * (kDim / 4) + lane;
#pragma unroll 16
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
            __syncthreads();                                              // everyone has read s_o
            if (warp > 0) {
#pragma unroll
                for (int h = 0; h < kGroup; ++h)
                    *reinterpret_cast<float4*>(&s_part[((warp - 1) * kGroup + h) * kDim + 4 * lane]) =
                        make_float4(r[h][0], r[h][1], r[h][2], r[h][3]);
            }
            __syncthreads();
            if (warp == 0) {
                __half* out_base = p.out + ((size_t)b * Hq + (size_t)kvh * kGroup) * kDim;
#pragma unroll
                for (int h = 0; h < kGroup; ++h) {
                    float4 v = make_float4(r[h][0], r[h][1], r[h][2], r[h][3]);
#pragma unroll
                    for (int w = 0; w < kAttnWarps - 1; ++w) {
                        const float4 a = *reinterpret_cast<const float4*>(&s_part[(w * kGroup + h) * kDim + 4 * lane]);
                        v.x += a.x; v.y += a.y; v.z += a.z; v.w += a.w;
                    }
                    const __half2 h01 = __floats2half2_rn(v.x, v.y), h23 = __floats2half2_rn(v.z, v.w);
                    uint2 pk;
                    pk.x = *reinterpret_cast<const uint32_t*>(&h01);
                    pk.y = *reinterpret_cast<const uint32_t*>(&h23);
                    *reinterpret_cast<uint2*>(out_base + h * kDim + 4 * lane) = pk;
                }
            }
            __syncthreads();                                              // s_res is free for the next segment
        }

        // ---- advance to the next pair ----
        f += seg_len;
        pg += seg_len;
        if (pg >= n_b && f < f_hi) {
            pg = 0;
            if (++kvh == H) {
                kvh = 0;
                do {
                    ++b;
                    seq_pg0 = ip(b);
                    n_b = ip(b + 1) - seq_pg0;
                } while (n_b <= 0 && b + 1 < p.B);
            }
        }
    }

    if constexpr (kCluster) {
        // ---- merge inside the cluster, through distributed shared memory ----
        // Every CTA holds the partial result of its pages in s_res[0] / s_m[0] / s_l[0]. After a cluster
        // barrier each CTA reads all kClusterCtas partials, merges them in rank order (every CTA gets the
        // same bits) and produces kDim / kClusterCtas of the output columns: out[:, c] = sum_i o[i] Pi_v[i][c].
        // No partial result goes through global memory and the rotation work is spread over the cluster;
        // each thread's 16 elements of Pi_v are fetched before the barrier.
        if (!waited) { pdl_begin(); waited = true; }           // a CTA without pages has not waited yet
        if (!have_partial) {
#pragma unroll
            for (int h = 0; h < kGroup; ++h) s_res[0][h][tid] = 0.f;
            if (tid < kGroup) {
                s_m[0][tid] = kNoRef;
                s_l[0][tid] = 0.f;
            }
        }
        constexpr int kCols = kDim / kClusterCtas;             // output columns per CTA (16 for 8 CTAs, 32 for 4)
        constexpr int kRowsPerPart = kDim / (kAttnThreads / kCols);   // rows of Pi_v per thread (16 / 32)
        static_assert(kCols == 16 || kCols == 32, "cluster of 8 or 4 CTAs");
        const int jcol = tid & (kCols - 1), ipart = tid / kCols;
        float pv[kRowsPerPart];
        {
            const float* src = p.Pi_v + (size_t)(ipart * kRowsPerPart) * kDim + crank * kCols + jcol;
#pragma unroll
            for (int ii = 0; ii < kRowsPerPart; ++ii) pv[ii] = __ldg(src + (size_t)ii * kDim);
        }
        asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
        asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");

        float* s_ml = &s_res[1][0][0];                         // [kClusterCtas][2 * kGroup]: m then l of every rank
        float* s_o = &s_res[2][0][0];                          // [kGroup][kDim] merged and normalised
        float* s_red = &s_res[3][0][0];                        // [kAttnWarps][kGroup][kCols]
        auto remote = [&](const void* local, unsigned rank) -> uint32_t {
            uint32_t r;
            asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_u32(local)), "r"(rank));
            return r;
        };
        auto ld_remote = [&](uint32_t addr) -> float {
            float v;
            asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(addr) : "memory");
            return v;
        };
        float ov[kClusterCtas][kGroup];
#pragma unroll
        for (int k = 0; k < kClusterCtas; ++k)
#pragma unroll
            for (int h = 0; h < kGroup; ++h) ov[k][h] = ld_remote(remote(&s_res[0][h][tid], k));
        if (tid < kClusterCtas * 2 * kGroup) {
            const int k = tid / (2 * kGroup), w = tid % (2 * kGroup);
            s_ml[tid] = ld_remote(remote(w < kGroup ? &s_m[0][w] : &s_l[0][w - kGroup], k));
        }
        __syncthreads();
#pragma unroll
        for (int h = 0; h < kGroup; ++h) {
            float m = s_ml[h];
#pragma unroll
            for (int k = 1; k < kClusterCtas; ++k) m = fmaxf(m, s_ml[k * 2 * kGroup + h]);
            float o = 0.f, l = 0.f;
#pragma unroll
            for (int k = 0; k < kClusterCtas; ++k) {
                const float fc = ex2_approx(s_ml[k * 2 * kGroup + h] - m);
                o = fmaf(fc, ov[k][h], o);
                l = fmaf(fc, s_ml[k * 2 * kGroup + kGroup + h], l);
            }
            s_o[h * kDim + tid] = l > 0.f ? o * (p.inv_alpha / l) : 0.f;
        }
        // this CTA has finished reading its neighbours' shared memory; nobody may leave before all have
        asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
        __syncthreads();
        float r[kGroup] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int ii = 0; ii < kRowsPerPart; ++ii) {
#pragma unroll
            for (int h = 0; h < kGroup; ++h) r[h] = fmaf(s_o[h * kDim + ipart * kRowsPerPart + ii], pv[ii], r[h]);
        }
        // with 16 columns a warp holds two parts (lanes 0..15 and 16..31): add them; then the four warps
        // through shared memory
        if (kCols == 16) {
#pragma unroll
            for (int h = 0; h < kGroup; ++h) r[h] += __shfl_xor_sync(0xffffffffu, r[h], 16);
        }
        if (lane < kCols) {
#pragma unroll
            for (int h = 0; h < kGroup; ++h) s_red[(warp * kGroup + h) * kCols + lane] = r[h];
        }
        __syncthreads();
        if (tid < kGroup * kCols) {
            const int h = tid / kCols, c = tid % kCols;
            float v = s_red[h * kCols + c];
#pragma unroll
            for (int w = 1; w < kAttnWarps; ++w) v += s_red[(w * kGroup + h) * kCols + c];
            p.out[((size_t)b * Hq + (size_t)kvh * kGroup + h) * kDim + crank * kCols + c] = __float2half_rn(v);
        }
        asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
    }
}
