// Causal attention of a chunk of prompt tokens over the packed pages, one query tile per CTA
// (included by tq_attn.cu, inside namespace leankv::{anonymous}).
//
// A CTA takes 32 consecutive query tokens of one kv head: 128 rows (token, GQA head), two 16-row MMA tiles per
// warp, which share every K / V operand fragment.
// It walks the sequence's pages up to the tile's last token; each page is fetched once (bulk copy,
// ring of 3), de-quantized once into shared memory as fp16 operands by the 128 threads (one 32-code
// unit each, the same byte-permute look-ups as the decode kernel) and then used by all four warps:
//   scores  S[32 rows][16 tokens] = Q''[32][128] . Khat^T    (mma.m16n8k16, Q'' = hi + lo fp16 halves
//                                                             of the rotated, pre-scaled query)
//   output  O[32 rows][128]      += P[32][16] . Vhat[16][128] (probabilities times value norms in fp16)
// with the usual online softmax per row in registers. So a page costs one de-quantization per 32
// query tokens instead of one per token, which is what the decode kernel run on prompt rows pays.
// When a tile has many pages they are cut into ranges handled by separate CTAs (grid z). Each CTA leaves its
// partial result in the rotated space (fp32 sums, maximum, denominator); tq_rot_rows_kernel<false> merges the
// ranges, normalises and applies Pi_V.

struct PrefillParams {
    const float* qprime;       // [T][Hq][128] rotated queries (Pi_K q), fp32
    float qscale;              // softmax scale * log2(e)
    float* o_part;             // [n_splits][T][Hq][128] un-normalised partial results in the rotated space
    float* ml_part;            // [n_splits][T][Hq][2]: running maximum (log2 units) and denominator of each partial
    int n_splits;              // the pages of a query tile are cut into this many ranges (grid z)
    uint32_t split_cum[9];     // range z of a tile with n pages = pages [n * cum[z] >> 16, n * cum[z+1] >> 16)
    const uint8_t* pool;
    int n_pages, H;
    const int32_t* seq_pages;  // the sequence's page ids in order
    int T, start_pos;
    uint32_t tl0, tl1, th0, th1;
    float inv_alpha;
    int* status;
};

// first page of range z of a tile with n_all pages (z = n_splits gives n_all)
__device__ __forceinline__ int split_begin(const PrefillParams& p, int n_all, int z) {
    return (int)(((unsigned long long)n_all * p.split_cum[z]) >> 16);
}

constexpr int kPfMt = 2;                       // 16-row MMA tiles per warp
constexpr int kPfTokens = 4 * 4 * kPfMt;       // query tokens per CTA: 4 warps x 4 tokens per tile x tiles
constexpr int kPfRows = kPfTokens * kGroup;    // 128 rows (token, GQA head)
constexpr int kPfStride = kDim + 8;            // halfs per row of the Q / K tiles (bank-conflict-free fragments)
constexpr int kPfVtStride = 24;                // halfs per row of the transposed V tile (16 tokens + padding)
constexpr int kPfStages = 3;
constexpr size_t kPfSmemBytes = (size_t)2 * kPfRows * kPfStride * 2      // Q'' hi and lo
                                + 2 * (size_t)kPage * kPfStride * 2       // K tiles [token][coord], two buffers
                                + 2 * (size_t)kDim * kPfVtStride * 2      // V tiles [coord][token], two buffers
                                + (size_t)kPfStages * 2 * kChunkBytes     // raw chunks
                                + 2 * 2 * kPage * sizeof(float)           // norms / alpha of K and V, two buffers
                                + kPfStages * 8;                          // mbarriers

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr));
}

__global__ void __launch_bounds__(kAttnThreads, 2) tq_prefill_attn_kernel(const PrefillParams p) {
    extern __shared__ __align__(128) uint8_t pf_smem[];
    uint8_t* s_raw = pf_smem;                                                   // [stages][K chunk | V chunk]
    __half* s_qh = reinterpret_cast<__half*>(s_raw + kPfStages * 2 * kChunkBytes);
    __half* s_ql = s_qh + kPfRows * kPfStride;
    // operands of a page, double-buffered: K tile, transposed V tile, norms / alpha per token
    constexpr int kKTile = kPage * kPfStride, kVTile = kDim * kPfVtStride;
    __half* s_k = s_ql + kPfRows * kPfStride;                                   // [2][kKTile]
    __half* s_vt = s_k + 2 * kKTile;                                            // [2][kVTile]
    float* s_kn = reinterpret_cast<float*>(s_vt + 2 * kVTile);                  // [2][kPage]
    float* s_vn = s_kn + 2 * kPage;                                             // [2][kPage]
    uint64_t* s_bar = reinterpret_cast<uint64_t*>(s_vn + 2 * kPage);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t = lane & 3;
    const int H = p.H, Hq = H * kGroup;
    const int n_tiles = (p.T + kPfTokens - 1) / kPfTokens;
    const int tile = n_tiles - 1 - (int)blockIdx.x;          // the tiles with the most pages start first
    const int kvh = blockIdx.y;
    const int tok0 = tile * kPfTokens;                       // first query token of the tile (chunk-relative)
    const int last_tok = min(tok0 + kPfTokens, p.T) - 1;
    const int n_all = (p.start_pos + last_tok) / kPage + 1;  // pages the tile's last token sees
    const int pg_lo = split_begin(p, n_all, blockIdx.z);
    const int n_pg = split_begin(p, n_all, blockIdx.z + 1) - pg_lo;                     // this CTA's share of them

    const uint32_t bar0 = smem_u32(s_bar);
    if (tid == 0) {
#pragma unroll
        for (int s = 0; s < kPfStages; ++s) mbar_init(bar0 + 8 * s, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    pdl_begin();
    __syncthreads();

    const size_t page_stride = (size_t)2 * H * kChunkBytes, kv_stride = (size_t)H * kChunkBytes;
    const uint8_t* pool_kvh = p.pool + (size_t)kvh * kChunkBytes;
    bool bad_page = false;
    auto issue = [&](int pg) {                               // thread 0 only
        int id = p.seq_pages[pg_lo + pg];
        if (id < 0 || id >= p.n_pages) {
            id = 0;
            bad_page = true;
        }
        const int s = pg % kPfStages;
        const uint8_t* src = pool_kvh + (size_t)id * page_stride;
        const uint32_t dst = smem_u32(s_raw + (size_t)s * 2 * kChunkBytes);
        mbar_expect_tx(bar0 + 8 * s, 2 * kChunkBytes);
        bulk_g2s(dst, src, kChunkBytes, bar0 + 8 * s);
        bulk_g2s(dst + kChunkBytes, src + kv_stride, kChunkBytes, bar0 + 8 * s);
    };
    if (tid == 0)
        for (int pg = 0; pg < min(kPfStages, n_pg); ++pg) issue(pg);

    // ---- the tile's queries: rotated, scaled, split into fp16 high and low halves ----
    for (int i = tid; i < kPfRows * (kDim / 4); i += kAttnThreads) {
        const int r = i / (kDim / 4), c4 = i % (kDim / 4);
        const int tok = tok0 + (r >> 2), head = r & 3;
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (tok < p.T)
            v = *reinterpret_cast<const float4*>(p.qprime + ((size_t)tok * Hq + (size_t)kvh * kGroup + head) * kDim + 4 * c4);
        const float x[4] = {v.x * p.qscale, v.y * p.qscale, v.z * p.qscale, v.w * p.qscale};
        __half hi[4], lo[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            hi[k] = __float2half_rn(x[k]);
            lo[k] = __float2half_rn(x[k] - __half2float(hi[k]));
        }
        *reinterpret_cast<uint2*>(s_qh + r * kPfStride + 4 * c4) = *reinterpret_cast<const uint2*>(hi);
        *reinterpret_cast<uint2*>(s_ql + r * kPfStride + 4 * c4) = *reinterpret_cast<const uint2*>(lo);
    }

    // The warp's rows: kPfMt tiles of 16 (token, head) rows, 4 tokens each; this lane holds rows g and g + 8 of
    // every tile. Tile mt covers tokens tok0 + 4 * (kPfMt * warp + mt) .. + 3.
    int qpos[kPfMt][2];
    float m_run[kPfMt][2], l_run[kPfMt][2];
    float acc[kPfMt][16][4];
#pragma unroll
    for (int mt = 0; mt < kPfMt; ++mt) {
        qpos[mt][0] = p.start_pos + tok0 + 4 * (kPfMt * warp + mt) + (g >> 2);   // position of row g's token
        qpos[mt][1] = qpos[mt][0] + 2;                                           // row g + 8: two tokens further
        m_run[mt][0] = m_run[mt][1] = kNoRef;
        l_run[mt][0] = l_run[mt][1] = 0.f;
#pragma unroll
        for (int j = 0; j < 16; ++j) acc[mt][j][0] = acc[mt][j][1] = acc[mt][j][2] = acc[mt][j][3] = 0.f;
    }
    __syncthreads();                                                     // the query tile is in shared memory
    // A fragments come from shared memory every page (ldmatrix.x4: rows 0-7 / 8-15 x k low / high of a tile)
    const uint32_t q_frag_off =
        (uint32_t)(((16 * kPfMt * warp + 8 * ((lane >> 3) & 1) + (lane & 7)) * kPfStride + 8 * (lane >> 4)) * 2);
    const uint32_t qh_frag = smem_u32(s_qh) + q_frag_off, ql_frag = smem_u32(s_ql) + q_frag_off;
    // ldmatrix row addresses of this lane (bytes, shared window): matrix L >> 3, row L & 7
    const uint32_t k_frag_addr =
        smem_u32(s_k + (8 * (lane >> 4) + (lane & 7)) * kPfStride + 8 * ((lane >> 3) & 1));
    const uint32_t v_frag_addr =
        smem_u32(s_vt + (8 * (lane >> 4) + (lane & 7)) * kPfVtStride + 8 * ((lane >> 3) & 1));
    bool failed = false;
    int fail_pg = 0;

    // De-quantize page pg of this CTA's range into operand buffer pg & 1: thread = one unit of 32 codes
    // (64 K units, 64 V units). Returns false if the page's copy did not arrive within the bound.
    auto dequant = [&](int pg) -> bool {
        const int s = pg % kPfStages, buf = pg & 1;
        if (!mbar_wait_bounded(bar0 + 8 * s, (uint32_t)((pg / kPfStages) & 1))) return false;
        const uint8_t* raw = s_raw + (size_t)s * 2 * kChunkBytes;
        const bool is_v = tid >= 64;
        const int ui = tid & 63;
        const Unit u = load_unit(reinterpret_cast<const uint32_t*>(raw + (is_v ? kChunkBytes : 0)), ui);
        uint32_t h2[16];                     // 32 fp16 values alpha * c[code], two per register, code order
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
        if (!is_v) {
            // K unit ui = 4 * token + quarter: coordinates 32 * quarter .. + 31 of the token, in order
            uint4* dst = reinterpret_cast<uint4*>(s_k + buf * kKTile + (ui >> 2) * kPfStride + 32 * (ui & 3));
#pragma unroll
            for (int q = 0; q < 4; ++q) dst[q] = make_uint4(h2[4 * q], h2[4 * q + 1], h2[4 * q + 2], h2[4 * q + 3]);
        } else {
            // V unit: coordinates 16 * grp .. + 15 of tokens 2 * pair and 2 * pair + 1, code 2 * c + parity:
            // register i holds the pair's two tokens of coordinate 16 * grp + i
            const int grp = (ui & 31) >> 2, pair = (ui & 3) + ((ui >> 5) << 2);
#pragma unroll
            for (int i = 0; i < 16; ++i)
                *reinterpret_cast<uint32_t*>(s_vt + buf * kVTile + (16 * grp + i) * kPfVtStride + 2 * pair) = h2[i];
        }
        if (tid < 2 * kPage) {
            const __half* nrm = reinterpret_cast<const __half*>(raw + (tid >= kPage ? kChunkBytes : 0) + kNormOffsetBytes);
            (tid >= kPage ? s_vn : s_kn)[buf * kPage + (tid & (kPage - 1))] = __half2float(nrm[tid & (kPage - 1)]) * p.inv_alpha;
        }
        return true;
    };

    // One barrier per page: it publishes the operands of page pg (written before it) and, since every warp
    // reaches it only after its work on page pg - 1, frees the other buffer for page pg + 1.
    bool got = n_pg > 0 ? dequant(0) : true;
    for (int pg = 0; pg < n_pg; ++pg) {
        if (__syncthreads_or(!got)) {
            failed = true;
            fail_pg = pg;
            break;
        }
        if (tid == 0 && pg + kPfStages < n_pg) issue(pg + kPfStages);      // page pg's raw chunk has been consumed
        const int buf = pg & 1;
        const float* kn = s_kn + buf * kPage;
        const float* vn = s_vn + buf * kPage;
        const uint32_t k_frag = k_frag_addr + (uint32_t)(buf * kKTile * 2);
        const uint32_t v_frag = v_frag_addr + (uint32_t)(buf * kVTile * 2);

        // ---- scores of this warp's rows against the page's 16 tokens ----
        float sc[kPfMt][2][4];
#pragma unroll
        for (int mt = 0; mt < kPfMt; ++mt)
#pragma unroll
            for (int j = 0; j < 2; ++j) sc[mt][j][0] = sc[mt][j][1] = sc[mt][j][2] = sc[mt][j][3] = 0.f;
#pragma unroll
        for (int ks = 0; ks < kDim / 16; ++ks) {
            // one ldmatrix brings the B fragments of both token tiles: matrices (tile 0, k low), (tile 0, k high),
            // (tile 1, k low), (tile 1, k high); lane L supplies row L & 7 of matrix L >> 3. They serve every
            // row tile of the warp.
            uint32_t kb[4];
            ldmatrix_x4(kb, k_frag + 2 * 16 * ks);
#pragma unroll
            for (int mt = 0; mt < kPfMt; ++mt) {
                uint32_t ah[4], al[4];
                ldmatrix_x4(ah, qh_frag + (uint32_t)((16 * mt * kPfStride + 16 * ks) * 2));
                ldmatrix_x4(al, ql_frag + (uint32_t)((16 * mt * kPfStride + 16 * ks) * 2));
                mma_16816(sc[mt][0], ah[0], ah[1], ah[2], ah[3], kb[0], kb[1]);
                mma_16816(sc[mt][0], al[0], al[1], al[2], al[3], kb[0], kb[1]);
                mma_16816(sc[mt][1], ah[0], ah[1], ah[2], ah[3], kb[2], kb[3]);
                mma_16816(sc[mt][1], al[0], al[1], al[2], al[3], kb[2], kb[3]);
            }
        }
        const int kbase = (pg_lo + pg) * kPage;
        const float vn0 = vn[2 * t], vn1 = vn[2 * t + 1], vn8 = vn[2 * t + 8], vn9 = vn[2 * t + 9];
        uint32_t pa[kPfMt][4];                  // P (times value norm / alpha) as A operands
#pragma unroll
        for (int mt = 0; mt < kPfMt; ++mt) {
            // key norm, causal mask (key position <= query position; every such position holds a token)
            float rmax0 = kNoRef, rmax1 = kNoRef;
#pragma unroll
            for (int j = 0; j < 2; ++j) {
#pragma unroll
                for (int c = 0; c < 2; ++c) {
                    const int tok = 8 * j + 2 * t + c;
                    const float knt = kn[tok];
                    const float v0 = kbase + tok <= qpos[mt][0] ? sc[mt][j][c] * knt : kNoRef;
                    const float v1 = kbase + tok <= qpos[mt][1] ? sc[mt][j][2 + c] * knt : kNoRef;
                    sc[mt][j][c] = v0;
                    sc[mt][j][2 + c] = v1;
                    rmax0 = fmaxf(rmax0, v0);
                    rmax1 = fmaxf(rmax1, v1);
                }
            }
            rmax0 = fmaxf(rmax0, __shfl_xor_sync(0xffffffffu, rmax0, 1));
            rmax0 = fmaxf(rmax0, __shfl_xor_sync(0xffffffffu, rmax0, 2));
            rmax1 = fmaxf(rmax1, __shfl_xor_sync(0xffffffffu, rmax1, 1));
            rmax1 = fmaxf(rmax1, __shfl_xor_sync(0xffffffffu, rmax1, 2));
            const float mn0 = fmaxf(m_run[mt][0], rmax0), mn1 = fmaxf(m_run[mt][1], rmax1);
            const float f0 = ex2_approx(m_run[mt][0] - mn0), f1 = ex2_approx(m_run[mt][1] - mn1);
            m_run[mt][0] = mn0;
            m_run[mt][1] = mn1;
            // probabilities; a masked entry is exactly 0, also while a row has seen nothing
            float pr[2][4];
            float sum0 = 0.f, sum1 = 0.f;
#pragma unroll
            for (int j = 0; j < 2; ++j) {
#pragma unroll
                for (int c = 0; c < 2; ++c) {
                    pr[j][c] = sc[mt][j][c] > 0.5f * kNoRef ? ex2_approx(sc[mt][j][c] - mn0) : 0.f;
                    pr[j][2 + c] = sc[mt][j][2 + c] > 0.5f * kNoRef ? ex2_approx(sc[mt][j][2 + c] - mn1) : 0.f;
                    sum0 += pr[j][c];
                    sum1 += pr[j][2 + c];
                }
            }
            l_run[mt][0] = l_run[mt][0] * f0 + sum0;   // per-lane partial sums; the quad is added up at the end
            l_run[mt][1] = l_run[mt][1] * f1 + sum1;
            if (__any_sync(0xffffffffu, f0 != 1.0f || f1 != 1.0f)) {      // a row's maximum moved: rescale its sums
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    acc[mt][j][0] *= f0; acc[mt][j][1] *= f0;
                    acc[mt][j][2] *= f1; acc[mt][j][3] *= f1;
                }
            }
            // tokens 2t, 2t+1 (tile 0) and 2t+8, 2t+9 (tile 1)
            pa[mt][0] = pack_h2(pr[0][0] * vn0, pr[0][1] * vn1);
            pa[mt][1] = pack_h2(pr[0][2] * vn0, pr[0][3] * vn1);
            pa[mt][2] = pack_h2(pr[1][0] * vn8, pr[1][1] * vn9);
            pa[mt][3] = pack_h2(pr[1][2] * vn8, pr[1][3] * vn9);
        }
#pragma unroll
        for (int j = 0; j < 16; j += 2) {
            // matrices (coords 8j.., tokens 0-7), (8j.., tokens 8-15), (8(j+1).., 0-7), (8(j+1).., 8-15)
            uint32_t vb[4];
            ldmatrix_x4(vb, v_frag + 2 * 8 * j * kPfVtStride);
#pragma unroll
            for (int mt = 0; mt < kPfMt; ++mt) {
                mma_16816(acc[mt][j], pa[mt][0], pa[mt][1], pa[mt][2], pa[mt][3], vb[0], vb[1]);
                mma_16816(acc[mt][j + 1], pa[mt][0], pa[mt][1], pa[mt][2], pa[mt][3], vb[2], vb[3]);
            }
        }
        if (pg + 1 < n_pg) got = dequant(pg + 1);        // into the other buffer, while slower warps finish page pg
    }
    if (failed || bad_page) {
        if (tid == 0) atomicOr(p.status, failed ? kStatusWaitTimeout : kStatusBadPage);
        if (failed) {
            // give the copies that were issued and not consumed a bounded chance to land before the CTA's
            // shared memory is handed to another CTA
            for (int q = fail_pg; q < min(fail_pg + kPfStages, n_pg); ++q)
                mbar_wait_bounded(bar0 + 8 * (q % kPfStages), (uint32_t)((q / kPfStages) & 1));
            return;
        }
    }

    // ---- this range's partial result, in the rotated space: sums, running maximum, denominator ----
    const size_t n_vec = (size_t)p.T * Hq;
    const int head = g & 3;
#pragma unroll
    for (int mt = 0; mt < kPfMt; ++mt) {
        float l0 = l_run[mt][0], l1 = l_run[mt][1];
        l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
        l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
        l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
        l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
        const int tokA = tok0 + 4 * (kPfMt * warp + mt) + (g >> 2), tokB = tokA + 2;
        const size_t vA = (size_t)tokA * Hq + (size_t)kvh * kGroup + head, vB = (size_t)tokB * Hq + (size_t)kvh * kGroup + head;
        float* oA = p.o_part + ((size_t)blockIdx.z * n_vec + vA) * kDim + 2 * t;
        float* oB = p.o_part + ((size_t)blockIdx.z * n_vec + vB) * kDim + 2 * t;
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            if (tokA < p.T) *reinterpret_cast<float2*>(oA + 8 * j) = make_float2(acc[mt][j][0], acc[mt][j][1]);
            if (tokB < p.T) *reinterpret_cast<float2*>(oB + 8 * j) = make_float2(acc[mt][j][2], acc[mt][j][3]);
        }
        if (t == 0) {
            if (tokA < p.T)
                *reinterpret_cast<float2*>(p.ml_part + ((size_t)blockIdx.z * n_vec + vA) * 2) = make_float2(m_run[mt][0], l0);
            if (tokB < p.T)
                *reinterpret_cast<float2*>(p.ml_part + ((size_t)blockIdx.z * n_vec + vB) * 2) = make_float2(m_run[mt][1], l1);
        }
    }
}

// ---- the same attention with both products on the fifth-generation tensor cores ----------------------------
// One CTA = 32 query tokens x 4 GQA heads = 128 rows = the M of tcgen05.mma; thread t owns row t, which is also
// accumulator lane t in tensor memory, so the online softmax needs no shuffles. Pages are taken two at a time
// (a block of 32 tokens): they are de-quantized into K-major blocked operand tiles (umma.cuh), one thread issues
//   S[128 x 32]  = Q''_h . K^T + Q''_l . K^T      16 MMAs (N = 32, K = 16) into one of two score buffers in tensor memory
// every thread reads its row of S (tcgen05.ld), applies key norm, causal mask and the running maximum, writes
// its 32 probabilities (times value norm, fp16) as a row of the P operand tile, and one thread issues
//   O[128 x 128] += P[128 x 32] . V[32 x 128]      2 MMAs (N = 128) into columns 64..191.
// The loop is software-pipelined: the keys of block b+1 are de-quantized (second K tile) and their score MMAs
// issued (second score buffer) before the softmax of block b, and the value MMAs of block b run under the key
// de-quantization of block b+2, so neither MMA group's latency is waited for in the open.
// The issuing thread runs on its own: the row warps tell it through two mbarriers (128 arrivals each) that a
// block's K / V tiles, or its P tile, are written, and hear back only through the MMA groups' commit barriers;
// among themselves the row warps meet once per block at a named barrier. So the ~2 000 cycles the single thread
// spends issuing 18 MMAs and 4 copies per block overlap the row warps' work instead of standing in their way.
// The running maximum only moves when a block exceeds it by more than kT5Slack (log2 units); then the rows of O
// are rescaled in tensor memory (tcgen05.ld / st), which is rare after the first blocks. Completion of each MMA
// group comes back through an mbarrier (tcgen05.commit) with a bounded wait. Output: the same partial results
// as tq_prefill_attn_kernel (un-normalised sums, maximum, denominator per row and page range).
constexpr int kT5Blk = 2;                          // pages per block
constexpr int kT5N = kT5Blk * kPage;               // 32 tokens per block
constexpr int kT5KChunksTok = kT5N / 8;            // 16-byte pieces along K for operands whose K is the token axis
constexpr float kT5Slack = 8.0f;
constexpr uint32_t kT5TmemCols = 256;              // S: 0..31 and 32..63, O: 64..191
constexpr int kT5Threads = 160;                    // four row warps + one warp whose first thread issues copies and MMAs
constexpr int kT5Issuer = 128;
constexpr int kT5Stages = 4;                      // raw page blocks in flight (three blocks of lead over their use)
constexpr int kT5KTileBytes = kT5N * kDim * 2;
// diagnostic status bits beside the time-out bit: the wait that ran out was for a page copy, the score MMAs, the value MMAs
constexpr int kT5WherePages = 0x10, kT5WhereScores = 0x20, kT5WhereValues = 0x40;
constexpr size_t kT5SmemBytes = 2 * (size_t)umma::kTileBytes             // Q'' high and low halves
                                + 2 * (size_t)kT5KTileBytes                // K tiles [token][coord], blocks b and b+1
                                + (size_t)kDim * kT5N * 2                  // V tile  [coord][token]
                                + (size_t)umma::kRows * kT5N * 2           // P tile  [row][token]
                                + (size_t)kT5Stages * kT5Blk * 2 * kChunkBytes   // raw chunks
                                + 2 * 4 * kT5N * sizeof(float) + 128;     // norms of four blocks; barriers

__global__ void __launch_bounds__(kT5Threads, 2) tq_prefill_t5_kernel(const PrefillParams p) {
    extern __shared__ __align__(1024) uint8_t t5_smem[];
    uint8_t* s_qh = t5_smem;
    uint8_t* s_ql = s_qh + umma::kTileBytes;
    uint8_t* s_k = s_ql + umma::kTileBytes;                     // B of S:  rows = tokens, K = coordinates (x 2)
    uint8_t* s_v = s_k + 2 * (size_t)kT5KTileBytes;             // B of O:  rows = coordinates, K = tokens
    uint8_t* s_p = s_v + (size_t)kDim * kT5N * 2;               // A of O:  rows = (token, head), K = tokens
    uint8_t* s_raw = s_p + (size_t)umma::kRows * kT5N * 2;      // [stages][page of the block][K chunk | V chunk]
    float* s_kn = reinterpret_cast<float*>(s_raw + (size_t)kT5Stages * kT5Blk * 2 * kChunkBytes);   // [block & 3][32]
    float* s_vn = s_kn + 4 * kT5N;
    // [0..3] raw stages, [4..5] S buffers, [6] O, [7] K / V tiles of a block written, [8] P tile written
    uint64_t* s_bar = reinterpret_cast<uint64_t*>(s_vn + 4 * kT5N);
    uint32_t* s_tmem = reinterpret_cast<uint32_t*>(s_bar + kT5Stages + 5);

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
    const uint32_t bar_o = bar0 + 8 * (kT5Stages + 2);
    const uint32_t bar_tiles = bar0 + 8 * (kT5Stages + 3), bar_probs = bar0 + 8 * (kT5Stages + 4);
    auto bar_raw = [&](int b) { return bar0 + 8u * (uint32_t)(b % kT5Stages); };
    auto bar_s = [&](int b) { return bar0 + 8u * (uint32_t)(kT5Stages + (b & 1)); };
    // block b is use number b / 4 of its raw stage and b / 2 of its score buffer: those uses' phase parities
    auto par_raw = [](int b) { return (uint32_t)((b / kT5Stages) & 1); };
    auto par2 = [](int b) { return (uint32_t)((b >> 1) & 1); };
    int where = 0;                                            // which bounded wait gave up (kT5Where* status bits)

    if (warp == 0) umma::tmem_alloc_n(smem_u32(s_tmem), kT5TmemCols);
    if (tid == 0) {
#pragma unroll
        for (int i = 0; i < kT5Stages + 3; ++i) mbar_init(bar0 + 8 * i, 1);
        mbar_init(bar_tiles, 128);
        mbar_init(bar_probs, 128);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    pdl_begin();
    umma::fence_before_sync();
    __syncthreads();
    umma::fence_after_sync();
    const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(s_tmem);
    const uint32_t tmem_o = tmem_base + 2 * kT5N;

    const size_t page_stride = (size_t)2 * H * kChunkBytes, kv_stride = (size_t)H * kChunkBytes;
    const uint8_t* pool_kvh = p.pool + (size_t)kvh * kChunkBytes;
    bool bad_page = false;
    int n_issued = 0;                                        // issuing thread: page blocks requested
    int next_id[kT5Blk] = {0, 0};                            // thread 0: page ids of the block issue() takes next
    auto load_ids = [&](int blk) {
#pragma unroll
        for (int i = 0; i < kT5Blk; ++i)
            next_id[i] = blk * kT5Blk + i < n_pg ? p.seq_pages[pg_lo + blk * kT5Blk + i] : 0;
    };
    auto issue = [&](int blk) {                              // thread 0: the block's (up to two) pages into stage blk % 4
        const int st = blk % kT5Stages;
        const int n_here = min(kT5Blk, n_pg - blk * kT5Blk);
        mbar_expect_tx(bar0 + 8 * st, (uint32_t)n_here * 2 * kChunkBytes);
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
            bulk_g2s(dst, src, kChunkBytes, bar0 + 8 * st);
            bulk_g2s(dst + kChunkBytes, src + kv_stride, kChunkBytes, bar0 + 8 * st);
        }
        n_issued = blk + 1;
        load_ids(blk + 1);                                   // calls come in block order: the ids are there by the next one
    };
    if (tid == kT5Issuer) {
        load_ids(0);
        for (int blk = 0; blk < min(kT5Stages, n_blk); ++blk) issue(blk);
    }

    // ---- the tile's queries: rotated, scaled, fp16 high and low halves, in the blocked operand layout ----
    for (int i = tid; i < umma::kRows * (kDim / 8); i += kT5Threads) {
        const int r = i % umma::kRows, k8 = i / umma::kRows;     // 8 lanes = 8 rows of one 128-byte core matrix
        const int tok = tok0 + (r >> 2), head = r & 3;
        float x[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        if (tok < p.T) {
            const float4* src = reinterpret_cast<const float4*>(p.qprime + ((size_t)tok * Hq + (size_t)kvh * kGroup + head) * kDim + 8 * k8);
            const float4 a = src[0], b = src[1];
            x[0] = a.x; x[1] = a.y; x[2] = a.z; x[3] = a.w; x[4] = b.x; x[5] = b.y; x[6] = b.z; x[7] = b.w;
        }
        __half hi[8], lo[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            const float v = x[e] * p.qscale;
            hi[e] = __float2half_rn(v);
            lo[e] = __float2half_rn(v - __half2float(hi[e]));
        }
        *reinterpret_cast<uint4*>(s_qh + umma::offset(r, k8)) = *reinterpret_cast<const uint4*>(hi);
        *reinterpret_cast<uint4*>(s_ql + umma::offset(r, k8)) = *reinterpret_cast<const uint4*>(lo);
    }

    // thread = one unit (32 codes) of page tid / 64 of the block: 32 fp16 values alpha * c[code], two per register
    const int pgi = tid >> 6, ui = tid & 63;
    auto unit_values = [&](const uint8_t* chunk, int unit, uint32_t (&h2)[16]) {
        const Unit u = load_unit(reinterpret_cast<const uint32_t*>(chunk), unit);
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
    };
    // norm of token j of block b (K or V chunk), times 1 / alpha; 0 for pages beyond the range
    auto norm_of = [&](int b, int j, bool is_v) -> float {
        const int pj = j >> 4;
        if (b * kT5Blk + pj >= n_pg) return 0.f;
        const uint8_t* rw = s_raw + ((size_t)(b % kT5Stages) * kT5Blk + pj) * 2 * kChunkBytes + (is_v ? kChunkBytes : 0);
        return __half2float(reinterpret_cast<const __half*>(rw + kNormOffsetBytes)[j & 15]) * p.inv_alpha;
    };
    auto dequant_keys = [&](int b) {                         // block b's keys -> K tile b & 1
        if (warp >= 4) return;
        uint32_t h2[16];
        // K unit 4 * token + quarter: coordinates 32 * quarter .. + 31 of the token = 4 pieces of row token;
        // 8 consecutive lanes take 8 consecutive tokens of one quarter, so a 16-byte store fills one core matrix
        const int ktok = ui & 15, kq = ui >> 4;
        unit_values(s_raw + ((size_t)(b % kT5Stages) * kT5Blk + pgi) * 2 * kChunkBytes, 4 * ktok + kq, h2);
        uint8_t* kt = s_k + (size_t)(b & 1) * kT5KTileBytes;
        const int trow = 16 * pgi + ktok, k8 = 4 * kq;
#pragma unroll
        for (int q = 0; q < 4; ++q)
            *reinterpret_cast<uint4*>(kt + umma::offset(trow, k8 + q)) = make_uint4(h2[4 * q], h2[4 * q + 1], h2[4 * q + 2], h2[4 * q + 3]);
        if (tid < kT5N) s_kn[(b & 3) * kT5N + tid] = norm_of(b, tid, false);
    };
    auto dequant_values = [&](int b) {                       // block b's values -> the V tile
        if (warp >= 4) return;
        uint32_t h2[16];
        unit_values(s_raw + ((size_t)(b % kT5Stages) * kT5Blk + pgi) * 2 * kChunkBytes + kChunkBytes, ui, h2);
        // V unit: coordinates 16 * grp .. + 15 of tokens 2 * pair, 2 * pair + 1: register i holds the pair's two
        // tokens of coordinate 16 * grp + i = 4 bytes of row (coordinate) along K (tokens). Lanes 4n .. 4n+3 hold
        // pairs 0..3 (or 4..7) of one group = the 8 tokens of a 16-byte piece: a 4 x 4 transpose between them
        // (per 4 registers) leaves lane p with the whole piece of coordinates 4j + p, stored with one instruction.
        const int grp = (ui & 31) >> 2, pl = ui & 3, half = ui >> 5;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            uint32_t* a = h2 + 4 * j;
#pragma unroll
            for (int c = 0; c < 4; c += 2) {                 // 2 x 2 blocks between lanes p, p ^ 1
                const uint32_t send = (pl & 1) ? a[c] : a[c + 1];
                const uint32_t got = __shfl_xor_sync(0xffffffffu, send, 1);
                if (pl & 1) a[c] = got; else a[c + 1] = got;
            }
#pragma unroll
            for (int c = 0; c < 2; ++c) {                    // then between lanes p, p ^ 2
                const uint32_t send = (pl & 2) ? a[c] : a[c + 2];
                const uint32_t got = __shfl_xor_sync(0xffffffffu, send, 2);
                if (pl & 2) a[c] = got; else a[c + 2] = got;
            }
            *reinterpret_cast<uint4*>(s_v + umma::offset_k(16 * grp + 4 * j + pl, 2 * pgi + half, kT5KChunksTok)) =
                make_uint4(a[0], a[1], a[2], a[3]);
        }
        if (tid < kT5N) s_vn[(b & 3) * kT5N + tid] = norm_of(b, tid, true);
    };
    auto issue_scores = [&](int b) {                         // thread 0: S(b) into score buffer b & 1
        const uint32_t qh = smem_u32(s_qh), ql = smem_u32(s_ql);
        const uint32_t kb = smem_u32(s_k) + (uint32_t)(b & 1) * kT5KTileBytes;
        const uint32_t ts = tmem_base + (uint32_t)(b & 1) * kT5N;
#pragma unroll
        for (int ks = 0; ks < kDim / 16; ++ks) {
            const uint32_t off = (uint32_t)ks * 2 * umma::kLbo;
            umma::mma_f16_n(ts, umma::desc(qh + off), umma::desc(kb + off), umma::idesc_n(kT5N), ks == 0 ? 0u : 1u);
            umma::mma_f16_n(ts, umma::desc(ql + off), umma::desc(kb + off), umma::idesc_n(kT5N), 1u);
        }
        umma::commit(bar_s(b));
    };

    const int row = tid;                                      // = accumulator lane
    const int lane0 = 32 * warp;
    const int qpos = p.start_pos + tok0 + (row >> 2);
    float m_ref = kNoRef, l_run = 0.f;
    bool failed = false;
    int n_pv = 0;                                             // value MMA groups committed

    // ---- prologue: keys of block 0, their score MMAs ----
    if (n_blk > 0 && warp < 4) {
        if (!umma::bar_wait(bar_raw(0), 0)) {
            failed = true;
            where |= kT5WherePages;
        }
        dequant_keys(0);
    }
    umma::fence_operands();
    umma::fence_before_sync();
    failed = __syncthreads_or(failed);                        // also publishes the query tiles
    umma::fence_after_sync();

    if (warp == 4) {
        // ------------------------------------------------------------------ the issuing thread
        if (tid == kT5Issuer && !failed && n_blk > 0) {
            issue_scores(0);
            for (int blk = 0; blk < n_blk; ++blk) {
                // K(blk + 1) and V(blk) are written, both halves of the raw stage of block blk consumed
                if (!umma::bar_wait(bar_tiles, (uint32_t)(blk & 1))) {
                    failed = true;
                    where |= kT5WherePages;
                    break;
                }
                umma::fence_after_sync();
                if (blk + 1 < n_blk) issue_scores(blk + 1);
                if (blk + kT5Stages < n_blk) issue(blk + kT5Stages);
                // P(blk) is written (and O rescaled where the reference moved)
                if (!umma::bar_wait(bar_probs, (uint32_t)(blk & 1))) {
                    failed = true;
                    where |= kT5WhereScores;
                    break;
                }
                umma::fence_after_sync();
                const uint32_t pb = smem_u32(s_p), vb = smem_u32(s_v);
#pragma unroll
                for (int kt = 0; kt < kT5N / 16; ++kt) {
                    const uint32_t off = (uint32_t)kt * 2 * umma::kLbo;
                    umma::mma_f16_n(tmem_o, umma::desc_k(pb + off, kT5KChunksTok), umma::desc_k(vb + off, kT5KChunksTok),
                                    umma::idesc_n(kDim), (blk == 0 && kt == 0) ? 0u : 1u);
                }
                umma::commit(bar_o);
            }
        }
    } else if (!failed) {
        // ------------------------------------------------------------------ the row warps
        // A wait that runs out makes the thread skip every later wait but not the barriers: all 128 threads
        // walk all blocks, so that nobody is left standing at the named barrier.
        for (int blk = 0; blk < n_blk; ++blk) {
            // (1) keys of the next block while S(blk) is on the tensor cores
            if (blk + 1 < n_blk) {
                if (!failed && !umma::bar_wait(bar_raw(blk + 1), par_raw(blk + 1))) {
                    failed = true;
                    where |= kT5WherePages;
                }
                dequant_keys(blk + 1);
            }
            // (2) values of this block: the previous block's value MMAs read the V and P tiles and must be done
            if (blk > 0) {
                if (!failed && !umma::bar_wait(bar_o, (uint32_t)((blk - 1) & 1))) {
                    failed = true;
                    where |= kT5WhereValues;
                }
                umma::fence_after_sync();
            }
            dequant_values(blk);
            umma::fence_operands();
            umma::fence_before_sync();
            umma::bar_arrive(bar_tiles);                                  // for the issuing thread
            asm volatile("bar.sync 1, 128;" ::: "memory");                // the block's value norms, for the other rows
            // (3) this thread's row of S(blk): key norm, causal mask, running maximum
            if (!failed && !umma::bar_wait(bar_s(blk), par2(blk))) {
                failed = true;
                where |= kT5WhereScores;
            }
            umma::fence_after_sync();
            {
                uint32_t sv[32];
                umma::ld32(sv, tmem_base + (uint32_t)(blk & 1) * kT5N, lane0, 0);
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
                // the reference only moves when the block exceeds it by more than the slack; the rows of O are then
                // rescaled in tensor memory (all lanes of a warp take part; lanes that do not move use factor 1)
                const bool move = bmax > m_ref + kT5Slack;
                const float m_new = move ? bmax : m_ref;
                const float f = move ? ex2_approx(m_ref - m_new) : 1.0f;
                if (__any_sync(0xffffffffu, move) && blk > 0) {
#pragma unroll
                    for (int c0 = 0; c0 < kDim; c0 += 32) {
                        uint32_t ov[32];
                        umma::ld32(ov, tmem_o, lane0, c0);
#pragma unroll
                        for (int i = 0; i < 32; ++i) ov[i] = __float_as_uint(__uint_as_float(ov[i]) * f);
                        umma::st32(ov, tmem_o, lane0, c0);
                    }
                }
                m_ref = m_new;
                l_run *= f;
                // probabilities (at most 2^slack) times value norm, fp16, as this row of the P operand
                {
                    float sum = 0.f;
                    __half2 ph[16];
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
                        ph[2 * j4] = __floats2half2_rn(pr[0] * n.x, pr[1] * n.y);
                        ph[2 * j4 + 1] = __floats2half2_rn(pr[2] * n.z, pr[3] * n.w);
                    }
                    l_run += sum;
#pragma unroll
                    for (int c = 0; c < kT5KChunksTok; ++c)
                        *reinterpret_cast<uint4*>(s_p + umma::offset_k(row, c, kT5KChunksTok)) = *reinterpret_cast<const uint4*>(ph + 4 * c);
                }
            }
            umma::fence_operands();
            umma::fence_before_sync();
            umma::bar_arrive(bar_probs);
            n_pv = blk + 1;
        }
    }
    if (!failed && n_pv > 0) {                                // row warps: the last value MMAs
        if (!umma::bar_wait(bar_o, (uint32_t)((n_pv - 1) & 1))) {
            failed = true;
            where |= kT5WhereValues;
        }
        umma::fence_after_sync();
    }
    failed = __syncthreads_or(failed);
    if (where != 0) atomicOr(p.status, where);
    if ((failed || bad_page) && tid == kT5Issuer) atomicOr(p.status, failed ? kStatusWaitTimeout : kStatusBadPage);
    if (failed && tid == kT5Issuer) {
        // give page copies that may still be in flight a bounded chance to land in this CTA's shared memory
        for (int b = max(0, n_issued - kT5Stages); b < n_issued; ++b) umma::bar_wait(bar_raw(b), par_raw(b));
    }

    // ---- this range's partial result for this thread's row ----
    // (tcgen05.ld is a warp-wide instruction: every lane takes part, rows beyond the chunk only skip the stores)
    const int tok = tok0 + (row >> 2), head = row & 3;
    const bool store = !failed && tok < p.T && warp < 4;
    const size_t n_vec = (size_t)p.T * Hq;
    const size_t v = (size_t)min(tok, p.T - 1) * Hq + (size_t)kvh * kGroup + head;
    float* dst = p.o_part + ((size_t)blockIdx.z * n_vec + v) * kDim;
    if (!failed && n_blk > 0 && warp < 4) {         // warp-uniform
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
    // tensor memory goes back before the CTA exits, whatever happened above
    umma::fence_before_sync();
    __syncthreads();
    if (warp == 0) umma::tmem_free_n(tmem_base, kT5TmemCols);
}

// Rotation of many vectors by one 128 x 128 matrix on the fifth-generation tensor cores (tcgen05): the matrix
// is split into fp16 high and low halves (B operands), the vectors likewise (A operands), both in shared memory
// in the blocked K-major layout the MMA's shared-memory descriptors address, and
//   out = a_h.M_h + a_h.M_l (+ a_l.M_h when the input is not exactly fp16)
// is accumulated in fp32 in tensor memory: the dropped low x low term is below 2^-22 of |a||M|. A CTA takes 128
// vectors (M = 128), N = 128, and issues 8 k-steps x 2 or 3 products of tcgen05.mma (128 x 128 x 16) from one
// elected thread; completion comes back through an mbarrier (tcgen05.commit), the four warps then read
// their 32 accumulator lanes with tcgen05.ld and store the result.
//   kForward:  out[v][j] = sum_k M[j][k] * in[v][k]     (query rotation, M = Pi_K; in fp16 (exact), out fp32)
//   !kForward: out[v][j] = sum_i in[v][i] * M[i][j]     (inverse value rotation, M = Pi_V; in = the page ranges'
//              partial results of the prefill kernel, merged and normalised here; out fp16)
//
// (operand layout and descriptors: umma.cuh)
constexpr int kRotRows = umma::kRows;
constexpr int kRotThreads = 256;
constexpr int kRotMaxSplits = 8;
constexpr size_t kRotSmemBytes = 4 * (size_t)umma::kTileBytes + (size_t)kRotRows * kRotMaxSplits * sizeof(float) + 16;

template <bool kForward>
__global__ void __launch_bounds__(kRotThreads) tq_rot_rows_kernel(const void* in, const float* ml_part, int n_splits,
                                                         const float* M, void* out, int n_vec, int* status) {
    extern __shared__ __align__(1024) uint8_t rot_smem[];
    uint8_t* s_bh = rot_smem;                                   // B high halves: [n = out coord][k], blocked
    uint8_t* s_bl = s_bh + umma::kTileBytes;
    uint8_t* s_ah = s_bl + umma::kTileBytes;                      // A high halves: [row][k], blocked
    uint8_t* s_al = s_ah + umma::kTileBytes;
    float* s_w = reinterpret_cast<float*>(s_al + umma::kTileBytes);         // [row][range]: merge weights
    uint64_t* s_bar = reinterpret_cast<uint64_t*>(s_w + kRotRows * kRotMaxSplits);
    uint32_t* s_tmem = reinterpret_cast<uint32_t*>(s_bar + 1);
    const int tid = threadIdx.x, warp = tid >> 5;
    const int v0 = blockIdx.x * kRotRows;

    if (warp == 0) umma::tmem_alloc(smem_u32(s_tmem));
    if (tid == 0) umma::bar_init(smem_u32(s_bar));
    // The matrix is a constant of the cache: stage it before the dependency wait. B[k][n] is M[n][k] for the
    // forward rotation (rows of M as they are) and M[k][n] for the inverse one (transposed copy).
    if (kForward) {
#pragma unroll 4
        for (int i = tid; i < kDim * (kDim / 8); i += kRotThreads) {
            const int n = i / (kDim / 8), k8 = i % (kDim / 8);
            const float4 w0 = __ldg(reinterpret_cast<const float4*>(M + (size_t)n * kDim + 8 * k8));
            const float4 w1 = __ldg(reinterpret_cast<const float4*>(M + (size_t)n * kDim + 8 * k8) + 1);
            const float x[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
            __half hi[8], lo[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                hi[e] = __float2half_rn(x[e]);
                lo[e] = __float2half_rn(x[e] - __half2float(hi[e]));
            }
            *reinterpret_cast<uint4*>(s_bh + umma::offset(n, k8)) = *reinterpret_cast<const uint4*>(hi);
            *reinterpret_cast<uint4*>(s_bl + umma::offset(n, k8)) = *reinterpret_cast<const uint4*>(lo);
        }
    } else {
        // thread (n, half) builds half of row n of the copy from column n of M (coalesced reads)
        const int n = tid & (kDim - 1);
#pragma unroll 2
        for (int k8 = (tid >> 7) * (kDim / 16); k8 < ((tid >> 7) + 1) * (kDim / 16); ++k8) {
            __half hi[8], lo[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                const float w = __ldg(M + (size_t)(8 * k8 + e) * kDim + n);
                hi[e] = __float2half_rn(w);
                lo[e] = __float2half_rn(w - __half2float(hi[e]));
            }
            *reinterpret_cast<uint4*>(s_bh + umma::offset(n, k8)) = *reinterpret_cast<const uint4*>(hi);
            *reinterpret_cast<uint4*>(s_bl + umma::offset(n, k8)) = *reinterpret_cast<const uint4*>(lo);
        }
    }
    pdl_begin();
    // ---- the tile's input rows as fp16 high and low halves ----
    if (!kForward) {
        // weights that merge the page ranges' partial results of a row: scale to the common maximum and
        // divide by the merged denominator (the value norms already carry 1 / alpha); one thread per row
        if (tid < kRotRows) {
        const int v = v0 + tid;
        float mz[kRotMaxSplits], lz[kRotMaxSplits];
        float m = kNoRef;
#pragma unroll
        for (int z = 0; z < kRotMaxSplits; ++z) {
            mz[z] = kNoRef;
            lz[z] = 0.f;
            if (z < n_splits && v < n_vec) {
                const float2 ml = *reinterpret_cast<const float2*>(ml_part + ((size_t)z * n_vec + v) * 2);
                mz[z] = ml.x;
                lz[z] = ml.y;
            }
            m = fmaxf(m, mz[z]);
        }
        float l = 0.f;
#pragma unroll
        for (int z = 0; z < kRotMaxSplits; ++z) {
            mz[z] = ex2_approx(mz[z] - m);
            l = fmaf(mz[z], lz[z], l);
        }
        const float inv = l > 0.f ? 1.0f / l : 0.f;
#pragma unroll
        for (int z = 0; z < kRotMaxSplits; ++z) s_w[tid * kRotMaxSplits + z] = mz[z] * inv;
        }
        __syncthreads();
    }
#pragma unroll 2
    for (int i = tid; i < kRotRows * (kDim / 8); i += kRotThreads) {
        const int r = i / (kDim / 8), k8 = i % (kDim / 8);
        const int v = v0 + r;
        float x[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        __half hi[8], lo[8];
        if (kForward) {
            uint4 raw = make_uint4(0u, 0u, 0u, 0u);
            if (v < n_vec) raw = *reinterpret_cast<const uint4*>(static_cast<const __half*>(in) + (size_t)v * kDim + 8 * k8);
            *reinterpret_cast<uint4*>(s_ah + umma::offset(r, k8)) = raw;          // exact fp16 input: no low half
        } else {
            if (v < n_vec) {
                const float* o_part = static_cast<const float*>(in);
                for (int z = 0; z < n_splits; ++z) {
                    const float f = s_w[r * kRotMaxSplits + z];
                    const float4* src = reinterpret_cast<const float4*>(o_part + ((size_t)z * n_vec + v) * kDim + 8 * k8);
                    const float4 o0 = src[0], o1 = src[1];
                    x[0] = fmaf(f, o0.x, x[0]); x[1] = fmaf(f, o0.y, x[1]); x[2] = fmaf(f, o0.z, x[2]); x[3] = fmaf(f, o0.w, x[3]);
                    x[4] = fmaf(f, o1.x, x[4]); x[5] = fmaf(f, o1.y, x[5]); x[6] = fmaf(f, o1.z, x[6]); x[7] = fmaf(f, o1.w, x[7]);
                }
            }
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                hi[e] = __float2half_rn(x[e]);
                lo[e] = __float2half_rn(x[e] - __half2float(hi[e]));
            }
            *reinterpret_cast<uint4*>(s_ah + umma::offset(r, k8)) = *reinterpret_cast<const uint4*>(hi);
            *reinterpret_cast<uint4*>(s_al + umma::offset(r, k8)) = *reinterpret_cast<const uint4*>(lo);
        }
    }
    // make the operands (written through the generic proxy) visible to the tensor core's async proxy
    umma::fence_operands();
    umma::fence_before_sync();
    __syncthreads();
    umma::fence_after_sync();
    const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(s_tmem);

    if (tid == 0) {
        const uint32_t ah = smem_u32(s_ah), al = smem_u32(s_al), bh = smem_u32(s_bh), bl = smem_u32(s_bl);
#pragma unroll
        for (int ks = 0; ks < kDim / 16; ++ks) {
            const uint32_t off = (uint32_t)ks * 2 * umma::kLbo;          // 16 k = two core matrices along K
            umma::mma_f16(tmem_base, umma::desc(ah + off), umma::desc(bh + off), ks == 0 ? 0u : 1u);
            umma::mma_f16(tmem_base, umma::desc(ah + off), umma::desc(bl + off), 1u);
            if (!kForward) umma::mma_f16(tmem_base, umma::desc(al + off), umma::desc(bh + off), 1u);
        }
        // the barrier is arrived on when every MMA issued above has completed
        umma::commit(smem_u32(s_bar));
    }
    const bool done = umma::bar_wait(smem_u32(s_bar), 0);
    umma::fence_after_sync();
    if (done) {
        // warp w reads accumulator lanes 32 (w % 4) .. + 31 = rows of the tile (the lanes a warp may touch follow
        // from its index modulo 4); warps 0-3 take columns 0-63, warps 4-7 columns 64-127; 32 columns per load
        const int lane0 = 32 * (warp & 3);
        const int v = v0 + lane0 + (tid & 31);
#pragma unroll
        for (int c0 = (warp >> 2) * (kDim / 2); c0 < ((warp >> 2) + 1) * (kDim / 2); c0 += 32) {
            uint32_t r[32];
            umma::ld32(r, tmem_base, lane0, c0);
            if (v < n_vec) {
                if (kForward) {
                    float4* o = reinterpret_cast<float4*>(static_cast<float*>(out) + (size_t)v * kDim + c0);
#pragma unroll
                    for (int q = 0; q < 8; ++q)
                        o[q] = make_float4(__uint_as_float(r[4 * q]), __uint_as_float(r[4 * q + 1]),
                                           __uint_as_float(r[4 * q + 2]), __uint_as_float(r[4 * q + 3]));
                } else {
                    uint4* o = reinterpret_cast<uint4*>(static_cast<__half*>(out) + (size_t)v * kDim + c0);
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        uint32_t pk[4];
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const __half2 h = __floats2half2_rn(__uint_as_float(r[8 * q + 2 * e]), __uint_as_float(r[8 * q + 2 * e + 1]));
                            pk[e] = *reinterpret_cast<const uint32_t*>(&h);
                        }
                        o[q] = make_uint4(pk[0], pk[1], pk[2], pk[3]);
                    }
                }
            }
        }
    } else if (tid == 0) {
        atomicOr(status, kStatusWaitTimeout);
    }
    // tensor memory goes back before the CTA exits, whatever happened above
    umma::fence_before_sync();
    __syncthreads();
    if (warp == 0) umma::tmem_free(tmem_base);
}
