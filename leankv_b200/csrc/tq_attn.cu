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
// mbarrier. Codes become tensor-core operands with byte-permute look-ups in 8-entry byte
// tables held in registers (one look-up yields four codes' bytes).
//  * Scores are integer MMAs (m16n8k32, s8): the centroids and the rotated query are 16-bit
//    fixed-point numbers split into a high and a low signed byte. The MMA's K dimension
//    carries 16 coordinates x {high, low} centroid byte, its rows the four GQA heads twice
//    (high x high, and high x low + low x high), its columns eight tokens; the low x low term
//    (2^-16 relative) is dropped. Integer sums are exact, so the only rounding on the key side is
//    the 16-bit representation of the query (per head, relative to its largest coordinate) and of
//    the centroids.
//  * The value sum is an fp16 MMA (m16n8k16): rows = coordinates, K = tokens, columns = heads.
//    The centroids enter scaled by a factor alpha chosen so that all eight are (almost) exactly
//    representable in fp16; probabilities times value norms are rounded to fp16, which is
//    independent from token to token and averages out over the sum. The score MMA's output
//    layout (heads in rows, tokens in columns) is exactly the value MMA's B operand layout, so
//    probabilities never move between lanes.
//
// Work is split over one wave of CTAs as equal shares of the flat list of all pages (see
// tq_attn_kernel.cuh); partial results of a (sequence, kv head) pair are merged, in CTA order, by
// the last CTA to arrive for it, which also applies the inverse value rotation.

#include <cmath>
#include <cstdlib>
#include <cstring>
#include <type_traits>

#include <algorithm>
#include <atomic>
#include <mutex>
#include <vector>

#include "common.cuh"
#include "tq_layout.cuh"
#include "umma.cuh"

namespace leankv {
namespace {

constexpr int kDim = LEANKV_TQ_DIM;
constexpr int kPage = LEANKV_TQ_PAGE_TOKENS;
constexpr int kAttnWarps = 4;
constexpr int kAttnThreads = kAttnWarps * 32;
constexpr int kStages = 4;
constexpr int kGroup = 4;                     // query heads per kv head
constexpr int kPartialFloats = kGroup * kDim + 2 * kGroup;
// Resident CTAs per SM: 4 (128 registers per thread, nothing spilled) by default, measured faster than
// the 96-register build (5 CTAs per SM, a few spilled bytes), which LEANKV_ATTN_OCC=5 selects.
int attn_occupancy() {
    static int occ = 0;
    if (occ == 0) {
        const char* e = std::getenv("LEANKV_ATTN_OCC");
        occ = (e != nullptr && e[0] == '5') ? 5 : 4;
    }
    return occ;
}
constexpr int kClusterMaxPages = 1024;        // 16384 tokens with 8 CTAs per pair (half that with 4): measured crossover near 32768
constexpr int kMinPagesPerCta = 4;            // short inputs use fewer CTAs rather than sub-page shares
constexpr float kFixedMax = 32512.0f;         // largest |value| of the 16-bit fixed-point operands (127 * 256)
constexpr int kSpinLimit = 1 << 20;
constexpr float kLog2e = 1.4426950408889634f;

// status bits written to the workspace status word
constexpr int kStatusWaitTimeout = 1;
constexpr int kStatusBadPage = 2;

struct AttnParams {
    const float* qprime;      // [B][Hq][128] rotated query Pi_k q
    float qscale;             // softmax scale * log2(e)
    __half* out;              // [B][Hq][128]
    const uint8_t* pool;
    int n_pages, H, B;
    const int32_t* indptr;
    const int32_t* indices;
    const int32_t* last_len;
    int flags;
    const float* Pi_v;
    uint32_t kh0, kh1, kl0, kl1;   // byte tables: high / low signed byte of round(c[0..7] / c_unit)
    float c_unit;                  // centroid value of one fixed-point unit
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

__device__ __forceinline__ void mma_s8_16832(int (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%0,%1,%2,%3};"
        : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// first MMA of a chain: the accumulator starts from the bias pattern (see kBiasBits) instead of being
// cleared by separate instructions
__device__ __forceinline__ void mma_s8_16832_bias(int (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    constexpr int kBias = 0x4B400000;
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%10,%10,%10,%10};"
        : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "r"(kBias));
}

__device__ __forceinline__ uint32_t pack_h2(float lo, float hi) {
    const __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&h);
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
// q_rot[v][j] = sum_k Pi_k[j][k] q[v][k] (ascending k). One CTA rotates kHeads consecutive query heads
// (the kGroup heads of one (sequence, kv head) pair; 16 heads when there are many rows, as in a prefill
// chunk), so each row of Pi_k is fetched once per kHeads heads.
template <int kHeads>
__global__ void __launch_bounds__(128) tq_qrot_kernel(const __half* q, const float* Pi_k, float* qprime) {
    __shared__ float s_q[kHeads][kDim];
    pdl_begin();
    const int v0 = blockIdx.x * kHeads, j = threadIdx.x;
#pragma unroll
    for (int h = 0; h < kHeads; ++h) s_q[h][j] = __half2float(q[(size_t)(v0 + h) * kDim + j]);
    __syncthreads();
    const float4* row = reinterpret_cast<const float4*>(Pi_k + (size_t)j * kDim);
    float acc[kHeads];
#pragma unroll
    for (int h = 0; h < kHeads; ++h) acc[h] = 0.f;
#pragma unroll (kHeads > kGroup ? 8 : 16)
    for (int k4 = 0; k4 < kDim / 4; ++k4) {
        const float4 pv = __ldg(row + k4);
#pragma unroll
        for (int h = 0; h < kHeads; ++h) {
            acc[h] = fmaf(pv.x, s_q[h][4 * k4 + 0], acc[h]);
            acc[h] = fmaf(pv.y, s_q[h][4 * k4 + 1], acc[h]);
            acc[h] = fmaf(pv.z, s_q[h][4 * k4 + 2], acc[h]);
            acc[h] = fmaf(pv.w, s_q[h][4 * k4 + 3], acc[h]);
        }
    }
#pragma unroll
    for (int h = 0; h < kHeads; ++h) qprime[(size_t)(v0 + h) * kDim + j] = acc[h];
}

// ---- main kernel -----------------------------------------------------------
#include "tq_attn_kernel.cuh"
#include "tq_prefill_kernel.cuh"
#include "tq_prefill_ws.cuh"

// ---- host side ---------------------------------------------------------------
struct AttnPlan {
    int n_ctas;
    size_t off_counters, off_qprime, off_partials, total;
};

// LEANKV_ATTN_CLUSTER=0 keeps a single sequence on the general kernel (partials through the workspace).
bool attn_cluster() {
    static int v = -1;
    if (v < 0) {
        const char* e = std::getenv("LEANKV_ATTN_CLUSTER");
        v = (e != nullptr && e[0] == '0') ? 0 : 1;
    }
    return v == 1;
}

// Largest page capacity (max_pages_per_seq) for which a single sequence uses the cluster variant; beyond it the
// general kernel's many CTAs win over the cluster's shorter tail. LEANKV_ATTN_CLUSTER_MAX_PAGES overrides.
int attn_cluster_max_pages() {
    static int v = -1;
    if (v < 0) {
        const char* e = std::getenv("LEANKV_ATTN_CLUSTER_MAX_PAGES");
        v = (e != nullptr && std::atoi(e) > 0) ? std::atoi(e) : kClusterMaxPages;
    }
    return v;
}

AttnPlan make_plan(int B, int Hq, int Hkv, int max_pages) {
    AttnPlan pl;
    if (max_pages < 1) max_pages = 1;
    const long long pairs = (long long)B * Hkv;
    // One wave of resident CTAs; inputs too short to give every CTA kMinPagesPerCta pages get fewer
    // (the kernel applies the same rule to the page count it finds on the device).
    const long long slots = (long long)sm_count() * attn_occupancy();
    long long want = pairs * ((max_pages + kMinPagesPerCta - 1) / kMinPagesPerCta);
    if (want < 1) want = 1;
    pl.n_ctas = (int)(want < slots ? want : slots);
    pl.off_counters = 256;
    pl.off_qprime = pl.off_counters + round_up(sizeof(int) * (size_t)pairs, 256);
    pl.off_partials = pl.off_qprime + round_up(sizeof(float) * (size_t)B * Hq * kDim, 256);
    // two partial results per CTA: the pair its share starts inside and the pair it ends inside
    pl.total = pl.off_partials + sizeof(float) * (size_t)pl.n_ctas * 2 * kPartialFloats;
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
    uint32_t kh0, kh1, kl0, kl1;
    float c_unit;
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
    // key side: 16-bit fixed point, split into a balanced low byte in [-128, 127] and a high byte
    float cmax = 0.f;
    for (int k = 0; k < 8; ++k) cmax = std::fmax(cmax, std::fabs(c[k]));
    const float unit = cmax > 0.f ? cmax / kFixedMax : 1.0f;
    uint32_t kh[2] = {0, 0}, kl[2] = {0, 0};
    for (int k = 0; k < 8; ++k) {
        const int ci = (int)std::lrintf(c[k] / unit);
        const int l8 = ((ci + 128) & 255) - 128;
        const int h8 = (ci - l8) / 256;
        kh[k >> 2] |= (uint32_t)(h8 & 255) << (8 * (k & 3));
        kl[k >> 2] |= (uint32_t)(l8 & 255) << (8 * (k & 3));
    }
    lut->kh0 = kh[0]; lut->kh1 = kh[1]; lut->kl0 = kl[0]; lut->kl1 = kl[1];
    lut->c_unit = unit;
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

// q (fp16, un-rotated) or q_rot (fp32, already Pi_k q) — exactly one of them is given.
static int attn_launch(const void* q, const float* q_rot, void* out, int B, int n_q_heads, int n_kv_heads,
                       const void* pool, int n_pages, const int32_t* kv_indptr,
                       const int32_t* kv_page_indices, const int32_t* kv_last_page_len,
                       int max_pages_per_seq, const float* Pi_k, const float* Pi_v, const float* centroids,
                       float scale, void* workspace, size_t workspace_bytes, int flags, void* stream) {
    if (B < 0 || n_q_heads <= 0 || n_kv_heads <= 0 || n_pages <= 0 || max_pages_per_seq < 0)
        return LEANKV_EINVAL;
    if (B == 0) return LEANKV_OK;
    if (n_q_heads != n_kv_heads * kGroup) return LEANKV_EUNSUPPORTED;
    if ((!q && !q_rot) || !out || !pool || !kv_indptr || !kv_page_indices || !kv_last_page_len || !Pi_v ||
        !centroids || !workspace || (q && !Pi_k))
        return LEANKV_EINVAL;
    if ((q && !aligned16(q)) || (q_rot && !aligned16(q_rot)) || !aligned16(out) || !aligned16(pool) ||
        (q && !aligned16(Pi_k)) || !aligned16(Pi_v) || !aligned16(workspace))
        return LEANKV_EALIGN;
    if (B > 65535 || n_kv_heads > 65535) return LEANKV_ELIMIT;
    if ((flags & ~LEANKV_ATTN_EARLY_FETCH) != 0) return LEANKV_EINVAL;
    const AttnPlan pl = make_plan(B, n_q_heads, n_kv_heads, max_pages_per_seq);
    if (workspace_bytes < pl.total) return LEANKV_EWORKSPACE;
    const Lut& lut = get_lut(centroids);

    char* ws = static_cast<char*>(workspace);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const float* qprime = q_rot;
    if (q != nullptr) {
        float* dst = reinterpret_cast<float*>(ws + pl.off_qprime);
        LEANKV_CUDA_TRY(launch_kernel(tq_qrot_kernel<kGroup>, dim3(B * n_kv_heads), dim3(128), 0, st,
                                      static_cast<const __half*>(q), Pi_k, dst));
        qprime = dst;
    }

    AttnParams p{};
    p.qprime = qprime;
    p.qscale = scale * kLog2e;
    p.out = static_cast<__half*>(out);
    p.pool = static_cast<const uint8_t*>(pool);
    p.n_pages = n_pages;
    p.H = n_kv_heads;
    p.B = B;
    p.indptr = kv_indptr;
    p.indices = kv_page_indices;
    p.last_len = kv_last_page_len;
    p.flags = flags;
    p.Pi_v = Pi_v;
    p.kh0 = lut.kh0; p.kh1 = lut.kh1; p.kl0 = lut.kl0; p.kl1 = lut.kl1;
    p.c_unit = lut.c_unit;
    p.tl0 = lut.tl0; p.tl1 = lut.tl1; p.th0 = lut.th0; p.th1 = lut.th1;
    p.inv_alpha = 1.0f / lut.alpha;
    p.partials = reinterpret_cast<float*>(ws + pl.off_partials);
    p.counters = reinterpret_cast<int*>(ws + pl.off_counters);
    p.status = reinterpret_cast<int*>(ws);
    // Few enough (sequence, kv head) pairs that a cluster of 8 or 4 CTAs per pair fits into one wave: the
    // pair's pages are split over its cluster and merged through distributed shared memory instead of the
    // workspace. (Every pair gets the same number of CTAs whatever its length; batches with many pairs take the
    // general kernel, whose flat split balances ragged lengths.)
    if (attn_cluster()) {
        const long long pairs = (long long)B * n_kv_heads, slots = (long long)sm_count() * 4;
        const int cs = pairs * 8 <= slots ? 8 : (pairs * 4 <= slots ? 4 : 0);
        if (cs != 0 && max_pages_per_seq <= attn_cluster_max_pages() * cs / 8) {
            if (cs == 8)
                LEANKV_CUDA_TRY(launch_cluster_kernel_ex(true, dim3(8), tq_decode_attn_kernel<4, 8>,
                                                         dim3((unsigned)pairs * 8), dim3(kAttnThreads), 0, st, p));
            else
                LEANKV_CUDA_TRY(launch_cluster_kernel_ex(true, dim3(4), tq_decode_attn_kernel<4, 4>,
                                                         dim3((unsigned)pairs * 4), dim3(kAttnThreads), 0, st, p));
            return LEANKV_OK;
        }
    }
    if (attn_occupancy() == 4)
        LEANKV_CUDA_TRY(launch_kernel_ex(true, tq_decode_attn_kernel<4, 0>, dim3(pl.n_ctas), dim3(kAttnThreads), 0, st, p));
    else
        LEANKV_CUDA_TRY(launch_kernel_ex(true, tq_decode_attn_kernel<5, 0>, dim3(pl.n_ctas), dim3(kAttnThreads), 0, st, p));
    return LEANKV_OK;
}

extern "C" int leankv_tq_decode_attn(const void* q, void* out, int B, int n_q_heads, int n_kv_heads,
                                     const void* pool, int n_pages, const int32_t* kv_indptr,
                                     const int32_t* kv_page_indices, const int32_t* kv_last_page_len,
                                     int max_pages_per_seq, const float* Pi_k, const float* Pi_v,
                                     const float* centroids, float scale, void* workspace,
                                     size_t workspace_bytes, void* stream) {
    if (!q) return LEANKV_EINVAL;
    return attn_launch(q, nullptr, out, B, n_q_heads, n_kv_heads, pool, n_pages, kv_indptr, kv_page_indices,
                       kv_last_page_len, max_pages_per_seq, Pi_k, Pi_v, centroids, scale, workspace,
                       workspace_bytes, 0, stream);
}

extern "C" int leankv_tq_decode_attn_rotated(const float* q_rot, void* out, int B, int n_q_heads,
                                             int n_kv_heads, const void* pool, int n_pages,
                                             const int32_t* kv_indptr, const int32_t* kv_page_indices,
                                             const int32_t* kv_last_page_len, int max_pages_per_seq,
                                             const float* Pi_v, const float* centroids, float scale,
                                             void* workspace, size_t workspace_bytes, int flags,
                                             void* stream) {
    if (!q_rot || (flags & ~LEANKV_ATTN_EARLY_FETCH) != 0) return LEANKV_EINVAL;
    return attn_launch(nullptr, q_rot, out, B, n_q_heads, n_kv_heads, pool, n_pages, kv_indptr,
                       kv_page_indices, kv_last_page_len, max_pages_per_seq, nullptr, Pi_v, centroids, scale,
                       workspace, workspace_bytes, flags, stream);
}

// ---- causal attention of a chunk of prompt tokens over the packed pages (tq_prefill_kernel.cuh) ----
static long long prefill_rows_pages(long long first_pos, long long n) {
    // sum over pos in [first_pos, first_pos + n) of pos / 16 + 1: page visits of the chunk's tokens
    auto upto = [](long long m) {
        const long long full = m / kPage, rest = m % kPage;
        return (long long)kPage * full * (full + 1) / 2 + rest * (full + 1);
    };
    return upto(first_pos + n) - upto(first_pos);
}

// The prefill attention's two products: tcgen05 with operands in shared memory (default), mma.sync
// (LEANKV_PREFILL_MMA=sync), or the warp-specialised tcgen05 form with query and probabilities in tensor memory
// (LEANKV_PREFILL_MMA=ws).
static int prefill_mode() {
    static int v = -1;
    if (v < 0) {
        const char* e = std::getenv("LEANKV_PREFILL_MMA");
        v = (e != nullptr && e[0] == 's') ? 0 : (e != nullptr && e[0] == 'w') ? 2 : 1;
    }
    return v;
}

struct TilePlan {
    int n_tiles, n_splits;
    size_t off_qprime, off_opart, off_ml, total;
};

// Where the page ranges of a tile begin (cumulative fractions in 1/65536). CTAs are handed to the SMs in grid
// order (tiles of one range first, longest tile first, then the next range), and with more CTAs than the
// 2 x SM-count that run at once equal ranges leave the last round of CTAs part-empty. Ranges that shrink
// geometrically put the short ones last, so the tail evens out. The ratio is picked by playing the schedule
// through on the host (every CTA goes to the slot that frees first; cost = pages + a fixed start-up) for
// equal ranges and three ratios; the last plan is remembered, since a model asks for it once per layer.
struct SplitPlan {
    uint32_t cum[9];
};
static SplitPlan plan_splits(const TilePlan& tp, int T, int start_pos, int Hkv) {
    static std::mutex mu;
    static long long last_key[4] = {-1, -1, -1, -1};
    static SplitPlan last_plan;
    std::lock_guard<std::mutex> lock(mu);
    const long long key[4] = {T, start_pos, Hkv, tp.n_splits};
    if (std::memcmp(key, last_key, sizeof(key)) == 0) return last_plan;
    const int s = tp.n_splits;
    const int slots = sm_count() * (prefill_mode() == 2 ? 1 : 2);
    auto fill = [&](double r, SplitPlan& sp) {
        double w[8], tot = 0.0, acc = 0.0;
        for (int z = 0; z < s; ++z) tot += (w[z] = std::pow(r, z));
        sp.cum[0] = 0;
        for (int z = 0; z < s; ++z) {
            acc += w[z];
            sp.cum[z + 1] = (uint32_t)std::llround(65536.0 * acc / tot);
        }
        sp.cum[s] = 65536;
        for (int z = s + 1; z <= 8; ++z) sp.cum[z] = 65536;
    };
    SplitPlan best;
    fill(1.0, best);
    const long long ctas = (long long)tp.n_tiles * Hkv * s;
    if (s > 1 && ctas > slots && ctas <= 16384) {
        const double ratios[4] = {1.0, 0.8, 0.7, 0.6};
        double best_t = 0.0;
        std::vector<double> heap;
        for (int c = 0; c < 4; ++c) {
            SplitPlan sp;
            fill(ratios[c], sp);
            heap.assign(slots, 0.0);                                  // min-heap of the times the slots free up
            auto cmp = [](double a, double b) { return a > b; };
            double t_end = 0.0;
            for (int z = 0; z < s; ++z)
                for (int y = 0; y < Hkv; ++y)
                    for (int x = 0; x < tp.n_tiles; ++x) {
                        const int tile = tp.n_tiles - 1 - x;
                        const long long last_tok = std::min<long long>((long long)tile * kPfTokens + kPfTokens, T) - 1;
                        const long long n_all = (start_pos + last_tok) / kPage + 1;
                        const long long n_pg = ((n_all * sp.cum[z + 1]) >> 16) - ((n_all * sp.cum[z]) >> 16);
                        std::pop_heap(heap.begin(), heap.end(), cmp);
                        heap.back() += 4.0 + (double)n_pg;
                        t_end = std::max(t_end, heap.back());
                        std::push_heap(heap.begin(), heap.end(), cmp);
                    }
            if (c == 0 || t_end < 0.98 * best_t) {                    // equal ranges unless a ratio clearly wins
                best_t = t_end;
                best = sp;
            }
        }
    }
    std::memcpy(last_key, key, sizeof(key));
    last_plan = best;
    return best;
}
// The pages of a query tile are cut into up to 8 ranges of at least ~16 pages, handled by separate CTAs, unless
// the (tile, kv head) pairs alone already make several waves: many short CTAs fill the SMs evenly although
// causal tiles differ in length (measured at 512 tokens after 3584: 2 ranges 366 us, 8 ranges 312 us).
static TilePlan make_tile_plan(int T, int start_pos, int Hq, int Hkv) {
    TilePlan tp;
    tp.n_tiles = (T + kPfTokens - 1) / kPfTokens;
    const long long ctas = (long long)tp.n_tiles * Hkv, slots = (long long)sm_count() * 2;
    long long s = ((long long)start_pos + T + kPage - 1) / kPage / 16;
    if (ctas >= 4 * slots) s = 1;
    if (s > 8) s = 8;
    if (s < 1) s = 1;
    tp.n_splits = (int)s;
    const size_t n_vec = (size_t)T * Hq;
    tp.off_qprime = 256;
    tp.off_opart = tp.off_qprime + round_up(sizeof(float) * n_vec * kDim, 256);
    tp.off_ml = tp.off_opart + round_up(sizeof(float) * n_vec * kDim * tp.n_splits, 256);
    tp.total = tp.off_ml + round_up(sizeof(float) * n_vec * 2 * tp.n_splits, 256);
    return tp;
}

extern "C" size_t leankv_tq_prefill_attn_workspace_bytes(int T, int start_pos, int n_q_heads,
                                                         int n_kv_heads) {
    if (T <= 0 || T > 65535 || start_pos < 0 || (long long)start_pos + T > (1ll << 24) || n_q_heads <= 0 ||
        n_kv_heads <= 0 || prefill_rows_pages(start_pos, T) > 0x7fffffffll)
        return 0;
    return make_tile_plan(T, start_pos, n_q_heads, n_kv_heads).total;
}

extern "C" int leankv_tq_prefill_attn(const void* q, void* out, int T, int start_pos, int n_q_heads,
                                      int n_kv_heads, const void* pool, int n_pages,
                                      const int32_t* seq_pages, const float* Pi_k, const float* Pi_v,
                                      const float* centroids, float scale, void* workspace,
                                      size_t workspace_bytes, void* stream) {
    if (T < 0 || start_pos < 0 || n_q_heads <= 0 || n_kv_heads <= 0 || n_pages <= 0) return LEANKV_EINVAL;
    if (T == 0) return LEANKV_OK;
    if (!q || !out || !pool || !seq_pages || !workspace || !Pi_k || !Pi_v || !centroids) return LEANKV_EINVAL;
    if (n_q_heads != n_kv_heads * kGroup) return LEANKV_EUNSUPPORTED;
    if (T > 65535 || (long long)start_pos + T > (1ll << 24)) return LEANKV_ELIMIT;
    if (prefill_rows_pages(start_pos, T) > 0x7fffffffll) return LEANKV_ELIMIT;     // page-table offsets are int32
    if (!aligned16(workspace) || !aligned16(q) || !aligned16(out) || !aligned16(pool) || !aligned16(Pi_k) ||
        !aligned16(Pi_v))
        return LEANKV_EALIGN;
    if (workspace_bytes < leankv_tq_prefill_attn_workspace_bytes(T, start_pos, n_q_heads, n_kv_heads))
        return LEANKV_EWORKSPACE;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const TilePlan tp = make_tile_plan(T, start_pos, n_q_heads, n_kv_heads);
    char* ws = static_cast<char*>(workspace);
    float* qprime = reinterpret_cast<float*>(ws + tp.off_qprime);
    float* o_part = reinterpret_cast<float*>(ws + tp.off_opart);
    float* ml_part = reinterpret_cast<float*>(ws + tp.off_ml);
    const Lut& lut = get_lut(centroids);
    static std::atomic<unsigned long long> attr_done{0};          // bit per device ordinal (< 64)
    int dev = 0;
    LEANKV_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return LEANKV_ELIMIT;
    if (((attr_done.load(std::memory_order_acquire) >> dev) & 1ull) == 0) {
        LEANKV_CUDA_TRY(cudaFuncSetAttribute(tq_prefill_attn_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             (int)kPfSmemBytes));
        LEANKV_CUDA_TRY(cudaFuncSetAttribute(tq_prefill_t5_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             (int)kT5SmemBytes));
        LEANKV_CUDA_TRY(cudaFuncSetAttribute(tq_prefill_ws_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             (int)kWsSmemBytes));
        LEANKV_CUDA_TRY(cudaFuncSetAttribute(tq_rot_rows_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             (int)kRotSmemBytes));
        LEANKV_CUDA_TRY(cudaFuncSetAttribute(tq_rot_rows_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             (int)kRotSmemBytes));
        attr_done.fetch_or(1ull << dev, std::memory_order_release);
    }
    const int n_vec = T * n_q_heads;
    const int rot_grid = (n_vec + kRotRows - 1) / kRotRows;
    LEANKV_CUDA_TRY(launch_kernel(tq_rot_rows_kernel<true>, dim3(rot_grid), dim3(kRotThreads), kRotSmemBytes, st, q,
                                  static_cast<const float*>(nullptr), 0, Pi_k, static_cast<void*>(qprime), n_vec,
                                  reinterpret_cast<int*>(ws)));
    PrefillParams p{};
    p.qprime = qprime;
    p.qscale = scale * kLog2e;
    p.o_part = o_part;
    p.ml_part = ml_part;
    p.n_splits = tp.n_splits;
    {
        const SplitPlan sp = plan_splits(tp, T, start_pos, n_kv_heads);
        std::memcpy(p.split_cum, sp.cum, sizeof(p.split_cum));
    }
    p.pool = static_cast<const uint8_t*>(pool);
    p.n_pages = n_pages;
    p.H = n_kv_heads;
    p.seq_pages = seq_pages;
    p.T = T;
    p.start_pos = start_pos;
    p.tl0 = lut.tl0; p.tl1 = lut.tl1; p.th0 = lut.th0; p.th1 = lut.th1;
    p.inv_alpha = 1.0f / lut.alpha;
    p.status = reinterpret_cast<int*>(ws);
    if (prefill_mode() == 2)
        LEANKV_CUDA_TRY(launch_kernel(tq_prefill_ws_kernel, dim3(tp.n_tiles, n_kv_heads, tp.n_splits),
                                      dim3(kWsThreads), kWsSmemBytes, st, p));
    else if (prefill_mode() == 1)
        LEANKV_CUDA_TRY(launch_kernel(tq_prefill_t5_kernel, dim3(tp.n_tiles, n_kv_heads, tp.n_splits),
                                      dim3(kT5Threads), kT5SmemBytes, st, p));
    else
        LEANKV_CUDA_TRY(launch_kernel(tq_prefill_attn_kernel, dim3(tp.n_tiles, n_kv_heads, tp.n_splits),
                                      dim3(kAttnThreads), kPfSmemBytes, st, p));
    LEANKV_CUDA_TRY(launch_kernel(tq_rot_rows_kernel<false>, dim3(rot_grid), dim3(kRotThreads), kRotSmemBytes, st,
                                  static_cast<const void*>(o_part), static_cast<const float*>(ml_part), tp.n_splits,
                                  Pi_v, out, n_vec, reinterpret_cast<int*>(ws)));
    return LEANKV_OK;
}

extern "C" int leankv_tq_decode_attn_status(const void* workspace, int* status) {
    if (!workspace || !status) return LEANKV_EINVAL;
    LEANKV_CUDA_TRY(cudaMemcpy(status, workspace, sizeof(int), cudaMemcpyDeviceToHost));
    return LEANKV_OK;
}
