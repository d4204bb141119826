// Paged decode attention straight from 3-bit TurboQuant codes (B200, sm_100a).
//
//   out[b][h] = softmax_t( scale * q[b][h] . k_hat[t] ) . v_hat[t]
//   k_hat[t] = nk[t] * (c[code_k[t]] @ Pi_k),  v_hat[t] = nv[t] * (c[code_v[t]] @ Pi_v)
//
// (the reconstruction of leankv/turboquant/quantizer.py:131-137 that
// leankv/turboquant/cache.py:169-189 materialises for every step). Nothing is
// de-quantized to memory here:
//   q . k_hat[t]      = nk[t] * ( (Pi_k q) . c[code_k[t]] )          -> rotate q once
//   sum_t p_t v_hat[t] = ( sum_t p_t nv[t] c[code_v[t]] ) @ Pi_v     -> rotate the sum once
//
// One warp owns one page (16 tokens) at a time. Its K and V chunks (800 bytes each) are
// brought into a per-warp shared-memory ring by bulk async copies that complete on an
// mbarrier. Codes become fp16 MMA operands with byte-permute look-ups: the eight
// centroids, scaled by a factor alpha chosen so that all of them are (almost) exactly
// representable in fp16, live in four registers used as 8-entry byte tables. Scores
// (16 tokens x 4 query heads) and the value sum (128 coordinates x 4 heads) are
// m16n8k16 tensor-core MMAs whose eight N columns carry the four GQA heads as fp16
// hi/lo pairs, so query and probability rounding does not limit accuracy.
//
// Split-KV: a CTA (4 warps) covers a range of pages; CTA partials are merged, in chunk
// order, by the last CTA to arrive for a (sequence, kv head), which also applies the
// inverse value rotation.

#include <cmath>
#include <cstring>

#include "common.cuh"
#include "tq_layout.cuh"

namespace leankv {
namespace {

constexpr int kDim = LEANKV_TQ_DIM;
constexpr int kAttnWarps = 4;
constexpr int kAttnThreads = kAttnWarps * 32;
constexpr int kStages = 4;
constexpr int kGroup = 4;                     // query heads per kv head
constexpr int kPartialFloats = kGroup * kDim + 2 * kGroup;
constexpr int kMaxChunks = 64;
constexpr int kSpinLimit = 1 << 20;
constexpr float kLog2e = 1.4426950408889634f;

// status bits written to the workspace status word
constexpr int kStatusWaitTimeout = 1;
constexpr int kStatusBadPage = 2;

struct AttnParams {
    const float* qprime;      // [B][Hq][128] rotated, pre-scaled query
    __half* out;              // [B][Hq][128]
    const uint8_t* pool;
    int n_pages, H, B;
    const int32_t* indptr;
    const int32_t* indices;
    const int32_t* last_len;
    int pages_per_cta, n_chunks;
    const float* Pi_v;
    uint32_t tl0, tl1, th0, th1;   // byte tables: low / high bytes of fp16(alpha * c[0..7])
    float inv_alpha;
    float* partials;
    int* counters;
    int* status;
};

// ---- PTX wrappers ----------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait: gives up after kSpinLimit polls instead of spinning forever.
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity) {
    for (int i = 0; i < kSpinLimit; ++i)
        if (mbar_try_wait(bar, parity)) return true;
    return false;
}
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
        "l"(src), "r"(bytes), "r"(bar)
        : "memory");
}
__device__ __forceinline__ void mma_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                          uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t pack_h2(float lo, float hi) {
    const __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&h);
}
// fp16 "hi" part of x, or the fp16 remainder x - hi ("lo" part).
__device__ __forceinline__ float split_part(float x, int part) {
    const float hi = __half2float(__float2half_rn(x));
    return part ? x - hi : hi;
}

struct Unit {
    uint32_t s[4];   // byte-permute selectors: 8 codes each, one per nibble
};
__device__ __forceinline__ Unit load_unit(const uint32_t* words, int ui) {
    const uint32_t w0 = words[ui], w1 = words[64 + ui], w2 = words[128 + ui];
    Unit u;
    u.s[0] = w0 & 0x77777777u;
    u.s[1] = w1 & 0x77777777u;
    u.s[2] = w2 & 0x77777777u;
    u.s[3] = ((w0 >> 3) & 0x11111111u) | ((w1 >> 2) & 0x22222222u) | ((w2 >> 1) & 0x44444444u);
    return u;
}

// ---- query rotation --------------------------------------------------------
__global__ void __launch_bounds__(128) tq_qrot_kernel(const __half* q, const float* Pi_k, float* qprime,
                                                      float qscale) {
    __shared__ float s_q[kDim];
    const int v = blockIdx.x, j = threadIdx.x;
    s_q[j] = __half2float(q[(size_t)v * kDim + j]);
    __syncthreads();
    const float4* row = reinterpret_cast<const float4*>(Pi_k + (size_t)j * kDim);
    float acc = 0.f;
#pragma unroll 8
    for (int k4 = 0; k4 < kDim / 4; ++k4) {
        const float4 pv = __ldg(row + k4);
        acc = fmaf(pv.x, s_q[4 * k4 + 0], acc);
        acc = fmaf(pv.y, s_q[4 * k4 + 1], acc);
        acc = fmaf(pv.z, s_q[4 * k4 + 2], acc);
        acc = fmaf(pv.w, s_q[4 * k4 + 3], acc);
    }
    qprime[(size_t)v * kDim + j] = acc * qscale;
}

// ---- main kernel -----------------------------------------------------------
__global__ void __launch_bounds__(kAttnThreads, 4) tq_decode_attn_kernel(const AttnParams p) {
    __shared__ __align__(128) uint8_t s_ring[kAttnWarps][kStages][2][kChunkBytes];
    __shared__ __align__(8) uint64_t s_bar[kAttnWarps][kStages];
    __shared__ float s_m[kAttnWarps][kGroup], s_l[kAttnWarps][kGroup];
    __shared__ __align__(16) float s_acc[kAttnWarps][kGroup][kDim];
    __shared__ __align__(16) float s_o[kGroup][kDim];
    __shared__ int s_last;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t = lane & 3;
    const int chunk = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
    const int Hq = p.H * kGroup;

    const int seq_pg0 = p.indptr[b];
    const int n_pages_b = p.indptr[b + 1] - seq_pg0;
    const int P = p.pages_per_cta;
    const int n_chunks_b = (n_pages_b + P - 1) / P;
    __half* out_base = p.out + ((size_t)b * Hq + (size_t)kvh * kGroup) * kDim;

    if (n_pages_b <= 0) {
        if (chunk == 0)
            for (int i = tid; i < kGroup * kDim; i += kAttnThreads) out_base[i] = __float2half_rn(0.f);
        return;
    }
    if (chunk >= n_chunks_b) return;

    int last_len = p.last_len[b];
    last_len = last_len < 1 ? 1 : (last_len > 16 ? 16 : last_len);
    const int cta_pg1 = min(n_pages_b, chunk * P + P);
    const int ppw = (P + kAttnWarps - 1) / kAttnWarps;
    const int w_pg0 = chunk * P + warp * ppw;
    const int n_my = max(0, min(cta_pg1, w_pg0 + ppw) - w_pg0);

    // Query as the B operand of the score MMA: column n = g is (head g/2, hi|lo part g%2);
    // k-step s covers rotated coordinates 32t + 4s .. +3.
    const int head = g >> 1, part = g & 1;
    uint32_t qf[8][2];
    {
        const float* qp = p.qprime + ((size_t)b * Hq + (size_t)kvh * kGroup + head) * kDim + 32 * t;
#pragma unroll
        for (int s = 0; s < 8; ++s) {
            const float4 v = *reinterpret_cast<const float4*>(qp + 4 * s);
            qf[s][0] = pack_h2(split_part(v.x, part), split_part(v.y, part));
            qf[s][1] = pack_h2(split_part(v.z, part), split_part(v.w, part));
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

    const int32_t* my_pages = p.indices + seq_pg0 + w_pg0;
    auto issue = [&](int i) {   // lane 0 only
        int page = my_pages[i];
        if (page < 0 || page >= p.n_pages) page = 0;   // flagged and masked at consume time
        const int s = i % kStages;
        const uint8_t* src_k = p.pool + (((size_t)page * 2 + 0) * p.H + kvh) * kChunkBytes;
        const uint8_t* src_v = p.pool + (((size_t)page * 2 + 1) * p.H + kvh) * kChunkBytes;
        mbar_expect_tx(bar0 + 8 * s, 2 * kChunkBytes);
        bulk_g2s(ring0 + s * 2 * kChunkBytes, src_k, kChunkBytes, bar0 + 8 * s);
        bulk_g2s(ring0 + s * 2 * kChunkBytes + kChunkBytes, src_v, kChunkBytes, bar0 + 8 * s);
    };
    int n_issued = 0;
    if (lane == 0)
        for (; n_issued < n_my && n_issued < kStages; ++n_issued) issue(n_issued);

    float m_run = -INFINITY, l_run = 0.f;
    float acc[8][4];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;

    int n_done = 0;
    bool failed = false;
    for (int i = 0; i < n_my; ++i) {
        const int s = i % kStages;
        // the verdict is made warp-uniform so that no lane is left behind at a shuffle
        if (!__all_sync(0xffffffffu, mbar_wait_bounded(bar0 + 8 * s, (i / kStages) & 1))) {
            failed = true;
            break;
        }
        n_done = i + 1;
        const int page = my_pages[i];
        const bool page_ok = page >= 0 && page < p.n_pages;
        if (!page_ok && lane == 0) atomicOr(p.status, kStatusBadPage);
        const int n_valid = !page_ok ? 0 : ((w_pg0 + i == n_pages_b - 1) ? last_len : 16);

        const uint8_t* stage = &s_ring[warp][s][0][0];
        const uint32_t* kw = reinterpret_cast<const uint32_t*>(stage);
        const __half* kn = reinterpret_cast<const __half*>(stage + kNormOffsetBytes);
        const uint32_t* vw = reinterpret_cast<const uint32_t*>(stage + kChunkBytes);
        const __half* vn = reinterpret_cast<const __half*>(stage + kChunkBytes + kNormOffsetBytes);

        // ---- scores: D[16 tokens][8 = 4 heads x (hi,lo)] ----
        float d[4] = {0.f, 0.f, 0.f, 0.f};
        {
            const Unit ua = load_unit(kw, lane), ub = load_unit(kw, 32 + lane);
#pragma unroll
            for (int q = 0; q < 8; ++q) {
                const uint32_t sa = ua.s[q >> 1] >> (16 * (q & 1));
                const uint32_t sb = ub.s[q >> 1] >> (16 * (q & 1));
                const uint32_t la = __byte_perm(p.tl0, p.tl1, sa), ha = __byte_perm(p.th0, p.th1, sa);
                const uint32_t lb = __byte_perm(p.tl0, p.tl1, sb), hb = __byte_perm(p.th0, p.th1, sb);
                mma_16816(d, __byte_perm(la, ha, 0x5140), __byte_perm(lb, hb, 0x5140),
                          __byte_perm(la, ha, 0x7362), __byte_perm(lb, hb, 0x7362), qf[q][0], qf[q][1]);
            }
        }
        const bool va = g < n_valid, vb = g + 8 < n_valid;
        const float sa = va ? (d[0] + d[1]) * __half2float(kn[g]) : -INFINITY;
        const float sb = vb ? (d[2] + d[3]) * __half2float(kn[g + 8]) : -INFINITY;
        float mt = fmaxf(sa, sb);
        mt = fmaxf(mt, __shfl_xor_sync(0xffffffffu, mt, 4));
        mt = fmaxf(mt, __shfl_xor_sync(0xffffffffu, mt, 8));
        mt = fmaxf(mt, __shfl_xor_sync(0xffffffffu, mt, 16));
        const float m_new = fmaxf(m_run, mt);
        if (n_valid > 0) {   // warp-uniform: false only for a page rejected as out of range
            const float m_safe = m_new == -INFINITY ? 0.f : m_new;
            if (__any_sync(0xffffffffu, m_new > m_run)) {
                const float f = exp2f(m_run - m_safe);   // 0 on the first page
                l_run *= f;
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    acc[j][0] *= f; acc[j][1] *= f; acc[j][2] *= f; acc[j][3] *= f;
                }
            }
            m_run = m_new;
            const float pa = va ? exp2f(sa - m_safe) : 0.f;
            const float pb = vb ? exp2f(sb - m_safe) : 0.f;
            l_run += pa + pb;
            const float wa = va ? pa * __half2float(vn[g]) : 0.f;
            const float wb = vb ? pb * __half2float(vn[g + 8]) : 0.f;

            // Probabilities as the B operand of the value MMA: rows = tokens, column n = g.
            const int src0 = (2 * t) * 4 + head, src1 = src0 + 4;
            const float x0 = __shfl_sync(0xffffffffu, wa, src0), x1 = __shfl_sync(0xffffffffu, wa, src1);
            const float x2 = __shfl_sync(0xffffffffu, wb, src0), x3 = __shfl_sync(0xffffffffu, wb, src1);
            const uint32_t b0 = pack_h2(split_part(x0, part), split_part(x1, part));
            const uint32_t b1 = pack_h2(split_part(x2, part), split_part(x3, part));

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
        if (lane == 0 && n_issued < n_my) {
            issue(n_issued);
            ++n_issued;
        }
    }
    if (failed) {
        // Give the copies still in flight a bounded chance to land before the CTA can exit.
        if (lane == 0) atomicOr(p.status, kStatusWaitTimeout);
        const int issued = __shfl_sync(0xffffffffu, n_issued, 0);
        for (int i = n_done; i < issued; ++i) mbar_wait_bounded(bar0 + 8 * (i % kStages), (i / kStages) & 1);
    }

    // ---- warp result -> shared memory ----
    l_run += __shfl_xor_sync(0xffffffffu, l_run, 4);
    l_run += __shfl_xor_sync(0xffffffffu, l_run, 8);
    l_run += __shfl_xor_sync(0xffffffffu, l_run, 16);
    if (g == 0) {
        s_m[warp][t] = m_run;
        s_l[warp][t] = l_run;
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        // rows g / g+8 of m-tile j are rotated coordinates 16g+2j / 16g+2j+1; columns 2t, 2t+1
        // are the hi and lo parts of head t.
        *reinterpret_cast<float2*>(&s_acc[warp][t][16 * g + 2 * j]) =
            make_float2(acc[j][0] + acc[j][1], acc[j][2] + acc[j][3]);
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
            const float mw = s_m[w][h];
            const float f = mw == -INFINITY ? 0.f : exp2f(mw - m);
            ov = fmaf(f, s_acc[w][h][tid], ov);
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
        const float* base = p.partials + (((size_t)b * p.H + kvh) * p.n_chunks) * kPartialFloats;
#pragma unroll
        for (int h = 0; h < kGroup; ++h) {
            float m = -INFINITY;
            for (int c = 0; c < n_chunks_b; ++c)
                m = fmaxf(m, ld_cg_f32(base + (size_t)c * kPartialFloats + kGroup * kDim + h));
            float ov = 0.f, lv = 0.f;
            for (int c = 0; c < n_chunks_b; ++c) {
                const float* pc = base + (size_t)c * kPartialFloats;
                const float mc = ld_cg_f32(pc + kGroup * kDim + h);
                const float f = mc == -INFINITY ? 0.f : exp2f(mc - m);
                ov = fmaf(f, ld_cg_f32(pc + h * kDim + tid), ov);
                lv = fmaf(f, ld_cg_f32(pc + kGroup * kDim + kGroup + h), lv);
            }
            o[h] = ov; lh[h] = lv;
        }
        if (tid == 0) p.counters[b * p.H + kvh] = 0;
    }

    // ---- normalise, undo the centroid scale, rotate back: out = o @ Pi_v ----
#pragma unroll
    for (int h = 0; h < kGroup; ++h) s_o[h][tid] = lh[h] > 0.f ? o[h] * (p.inv_alpha / lh[h]) : 0.f;
    __syncthreads();
    float r[kGroup] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 8
    for (int i = 0; i < kDim; ++i) {
        const float pv = __ldg(p.Pi_v + (size_t)i * kDim + tid);
#pragma unroll
        for (int h = 0; h < kGroup; ++h) r[h] = fmaf(s_o[h][i], pv, r[h]);
    }
#pragma unroll
    for (int h = 0; h < kGroup; ++h) out_base[h * kDim + tid] = __float2half_rn(r[h]);
}

// ---- host side ---------------------------------------------------------------
struct AttnPlan {
    int pages_per_cta, n_chunks;
    size_t off_counters, off_qprime, off_partials, total;
};

AttnPlan make_plan(int B, int Hq, int Hkv, int max_pages) {
    AttnPlan pl;
    if (max_pages < 1) max_pages = 1;
    const long long pairs = (long long)B * Hkv;
    long long slots = (long long)sm_count() * 4;
    long long nc = slots / (pairs > 0 ? pairs : 1);
    if (nc < 1) nc = 1;
    const int by_pages = (max_pages + kAttnWarps - 1) / kAttnWarps;   // at least one page per warp
    if (nc > by_pages) nc = by_pages;
    if (nc > kMaxChunks) nc = kMaxChunks;
    pl.pages_per_cta = (int)((max_pages + nc - 1) / nc);
    pl.n_chunks = (max_pages + pl.pages_per_cta - 1) / pl.pages_per_cta;
    pl.off_counters = 256;
    pl.off_qprime = pl.off_counters + round_up(sizeof(int) * (size_t)pairs, 256);
    pl.off_partials = pl.off_qprime + round_up(sizeof(float) * (size_t)B * Hq * kDim, 256);
    pl.total = pl.off_partials +
               (pl.n_chunks > 1 ? sizeof(float) * (size_t)pairs * pl.n_chunks * kPartialFloats : 0);
    return pl;
}

// fp16 helpers on the host (round-to-nearest-even through the CUDA host intrinsics).
inline uint16_t f2h_bits(float f) {
    const __half h = __float2half_rn(f);
    uint16_t b;
    std::memcpy(&b, &h, 2);
    return b;
}
inline float h_bits2f(uint16_t b) {
    __half h;
    std::memcpy(&h, &b, 2);
    return __half2float(h);
}

struct Lut {
    float centroids[8];
    uint32_t tl0, tl1, th0, th1;
    float alpha;
    bool valid;
};

// Scale factor alpha in [1,2) minimising the worst relative fp16 rounding error of
// alpha*c[i]; the codebook then enters the tensor cores with ~1e-5 relative error
// instead of 2^-11.
void build_lut(const float* c, Lut* lut) {
    double best_err = 1e30;
    float best_alpha = 1.f;
    for (int i = 0; i < 65536; ++i) {
        const float alpha = 1.0f + (float)i / 65536.0f;
        double worst = 0.0;
        for (int k = 0; k < 8; ++k) {
            const float v = alpha * c[k];
            if (v == 0.f) continue;
            const double e = std::fabs((double)h_bits2f(f2h_bits(v)) / (double)v - 1.0);
            if (e > worst) worst = e;
        }
        if (worst < best_err) {
            best_err = worst;
            best_alpha = alpha;
        }
    }
    uint32_t lo[2] = {0, 0}, hi[2] = {0, 0};
    for (int k = 0; k < 8; ++k) {
        const uint16_t hb = f2h_bits(best_alpha * c[k]);
        lo[k >> 2] |= (uint32_t)(hb & 0xff) << (8 * (k & 3));
        hi[k >> 2] |= (uint32_t)(hb >> 8) << (8 * (k & 3));
    }
    std::memcpy(lut->centroids, c, sizeof(float) * 8);
    lut->tl0 = lo[0]; lut->tl1 = lo[1]; lut->th0 = hi[0]; lut->th1 = hi[1];
    lut->alpha = best_alpha;
    lut->valid = true;
}

const Lut& get_lut(const float* c) {
    static thread_local Lut cache = {};
    if (!cache.valid || std::memcmp(cache.centroids, c, sizeof(float) * 8) != 0) build_lut(c, &cache);
    return cache;
}

}  // namespace
}  // namespace leankv

using namespace leankv;

extern "C" size_t leankv_tq_decode_attn_workspace_bytes(int B, int n_q_heads, int n_kv_heads,
                                                        int max_pages_per_seq) {
    if (B <= 0 || n_q_heads <= 0 || n_kv_heads <= 0) return 0;
    return make_plan(B, n_q_heads, n_kv_heads, max_pages_per_seq).total;
}

extern "C" int leankv_tq_decode_attn(const void* q, void* out, int B, int n_q_heads, int n_kv_heads,
                                     const void* pool, int n_pages, const int32_t* kv_indptr,
                                     const int32_t* kv_page_indices, const int32_t* kv_last_page_len,
                                     int max_pages_per_seq, const float* Pi_k, const float* Pi_v,
                                     const float* centroids, float scale, void* workspace,
                                     size_t workspace_bytes, void* stream) {
    if (B < 0 || n_q_heads <= 0 || n_kv_heads <= 0 || n_pages <= 0 || max_pages_per_seq < 0)
        return LEANKV_EINVAL;
    if (B == 0) return LEANKV_OK;
    if (n_q_heads != n_kv_heads * kGroup) return LEANKV_EUNSUPPORTED;
    if (!q || !out || !pool || !kv_indptr || !kv_page_indices || !kv_last_page_len || !Pi_k || !Pi_v ||
        !centroids || !workspace)
        return LEANKV_EINVAL;
    if (!aligned16(q) || !aligned16(out) || !aligned16(pool) || !aligned16(Pi_k) || !aligned16(Pi_v) ||
        !aligned16(workspace))
        return LEANKV_EALIGN;
    if (B > 65535 || n_kv_heads > 65535) return LEANKV_ELIMIT;
    const AttnPlan pl = make_plan(B, n_q_heads, n_kv_heads, max_pages_per_seq);
    if (workspace_bytes < pl.total) return LEANKV_EWORKSPACE;
    const Lut& lut = get_lut(centroids);

    char* ws = static_cast<char*>(workspace);
    float* qprime = reinterpret_cast<float*>(ws + pl.off_qprime);
    cudaStream_t st = static_cast<cudaStream_t>(stream);

    tq_qrot_kernel<<<B * n_q_heads, 128, 0, st>>>(static_cast<const __half*>(q), Pi_k, qprime,
                                                  scale * kLog2e / lut.alpha);
    LEANKV_CUDA_TRY(cudaGetLastError());

    AttnParams p{};
    p.qprime = qprime;
    p.out = static_cast<__half*>(out);
    p.pool = static_cast<const uint8_t*>(pool);
    p.n_pages = n_pages;
    p.H = n_kv_heads;
    p.B = B;
    p.indptr = kv_indptr;
    p.indices = kv_page_indices;
    p.last_len = kv_last_page_len;
    p.pages_per_cta = pl.pages_per_cta;
    p.n_chunks = pl.n_chunks;
    p.Pi_v = Pi_v;
    p.tl0 = lut.tl0; p.tl1 = lut.tl1; p.th0 = lut.th0; p.th1 = lut.th1;
    p.inv_alpha = 1.0f / lut.alpha;
    p.partials = reinterpret_cast<float*>(ws + pl.off_partials);
    p.counters = reinterpret_cast<int*>(ws + pl.off_counters);
    p.status = reinterpret_cast<int*>(ws);
    dim3 grid(pl.n_chunks, n_kv_heads, B);
    tq_decode_attn_kernel<<<grid, kAttnThreads, 0, st>>>(p);
    LEANKV_CUDA_TRY(cudaGetLastError());
    return LEANKV_OK;
}

extern "C" int leankv_tq_decode_attn_status(const void* workspace, int* status) {
    if (!workspace || !status) return LEANKV_EINVAL;
    LEANKV_CUDA_TRY(cudaMemcpy(status, workspace, sizeof(int), cudaMemcpyDeviceToHost));
    return LEANKV_OK;
}
