// TEAL activation-sparse GEMV for batch-1 decode on B200.
//
// y[n] = sum_{z : |x[z]| > t} Wt[z][n] * x[z]        (Wt is [Z][N], rows contiguous)
//
// Work decomposition: a CTA owns 256 output columns (one 16-byte load per lane per row)
// and a contiguous range of input channels. It tests the threshold on its range,
// compacts the surviving channels with warp ballot/popc into an ordered list in shared
// memory, and its 8 warps stream the listed weight rows round-robin, 8 independent
// 16-byte loads in flight per lane. Split-K partials go to a workspace; the last CTA to
// arrive for a column slice sums them in split order, so the result does not depend on
// arrival order and no floating-point atomics are used.
//
// The same kernel also serves: per-segment thresholds (fused q/k/v), bias, residual add, the fused
// gate/up SwiGLU (template flag), RMSNorm of the input row fused into the prologue, and the
// tensor-parallel form in which the finishing CTA sums the ranks' partial products over peer
// memory before it writes y.
//
// Arithmetic follows the reference's B=1 path (leankv/teal/kernels/sparse_gemv.py:71-87:
// fp16 operands widened to fp32, fp32 sums) and the mask of leankv/teal/sparse_fns.py:36
// (strict '>' against the threshold rounded to fp16).

#include "common.cuh"

namespace leankv {
namespace {

constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;
constexpr int kColsPerCta = 256;       // 32 lanes x 8 fp16
constexpr int kLaneSlots = 4;          // threshold tests per lane during compaction
constexpr int kMaxRowsPerSplit = kWarps * 32 * kLaneSlots;  // 1024
constexpr int kMaxSplits = 128;
constexpr int kMaxSplitsNarrow = 40;   // = kWarps x the merge's load batch: the last CTA sums a slice in one round trip
constexpr int kCtasPerSm = 4;
constexpr size_t kCounterAreaBytes = 16384;   // counters of up to 4096 column slices (N <= 1 048 576)

struct GemvParams {
    const __half* Wt;
    const __half* Wt2;   // up_proj weights (SwiGLU only)
    const __half* x;
    __half* y;
    const __half* bias;
    const __half* residual;
    float* partials;
    int* counters;
    unsigned long long* active_elems;
    int N, Z;
    int n_slices, k_splits, rows_per_split;
    int prefetch_rows;   // weight rows of its range a CTA asks into L2 before it waits for the previous kernel
    int n_segments;
    int seg_end[LEANKV_MAX_SEGMENTS];
    float thr[LEANKV_MAX_SEGMENTS];
    float thr_up;        // SwiGLU: thr[0] masks gate, thr_up masks up
    const __half* norm_w;   // if set, x is an un-normalised row h and the kernel uses
    float norm_eps;         // x[z] = norm_w[z] * fp16(h[z] * rsqrt(mean(h^2) + eps))  (RMSNorm fused in)
    // All-reduce of the row-parallel partial products over peer memory (xw = 0: off).
    // xrecv[r]: rank r's receive area for this launch's slot, as mapped into this process:
    // 64-bit words [world][npad] indexed by source rank, each {fp32 value, epoch}.
    int xw, xrank, xlimit;
    unsigned long long* xrecv[LEANKV_MAX_RANKS];
    const int* xepoch;
    int* xstatus;
};

// One 64-bit access carries a value together with the epoch that marks it as arrived, so the
// exchange needs no fence and no separate flag (a scalar 64-bit access is never torn).
__device__ __forceinline__ void st_relaxed_sys_u64(unsigned long long* p, unsigned long long v) {
    asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ unsigned long long ld_relaxed_sys_u64(const unsigned long long* p) {
    unsigned long long v;
    asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}

struct GemvPlan {
    int n_slices, k_splits, rows_per_split;
    size_t counter_bytes, partial_bytes;
};

// How many weight rows of its range a CTA asks into L2 ahead of the dependency wait: LEANKV_GEMV_PREFETCH_KB
// kilobytes per CTA (default 32; 0 = off), at most LEANKV_GEMV_PREFETCH_PCT per cent of the range (default 25).
// Measured on the Mistral-7B-shape decode step: off 427.2 tok/s, 16 KB 435.5, 32 KB 437.6 (25 %: 438.1), 48 KB 434.0.
static int prefetch_rows(int rows_per_split, int arrays) {
    static int kb = -1, pct = -1;
    if (kb < 0) {
        const char* e = std::getenv("LEANKV_GEMV_PREFETCH_KB");
        kb = e != nullptr ? std::max(0, std::min(512, std::atoi(e))) : 32;
        const char* f = std::getenv("LEANKV_GEMV_PREFETCH_PCT");
        pct = f != nullptr ? std::max(0, std::min(100, std::atoi(f))) : 25;
    }
    const int by_bytes = kb * 1024 / (kColsPerCta * 2 * arrays);
    const int by_share = (int)((long long)rows_per_split * pct / 100);
    return std::min(std::min(by_bytes, by_share), kThreads / arrays);
}

GemvPlan make_plan(int N, int Z, int arrays) {
    GemvPlan pl;
    pl.n_slices = (N + kColsPerCta - 1) / kColsPerCta;
    // resident CTAs per SM: 4 for the plain kernel (64 registers), 3 for the SwiGLU kernel (80)
    int target = sm_count() * (arrays == 2 ? 3 : kCtasPerSm);
    int ks = target / pl.n_slices;
    if (ks < 1) ks = 1;
    int by_rows = Z / 32;            // keep at least ~32 input channels per split
    if (by_rows < 1) by_rows = 1;
    if (ks > by_rows) ks = by_rows;
    // Narrow matrices (a tensor-parallel rank's share) would otherwise be cut into ~100 splits of a few
    // rows each, and the time goes into merging them: measured 8.6 -> 6.8 us for 768 x 4096.
    const int max_splits = pl.n_slices <= 8 ? kMaxSplitsNarrow : kMaxSplits;
    if (ks > max_splits) ks = max_splits;
    int rows = (Z + ks - 1) / ks;
    if (rows > kMaxRowsPerSplit) rows = kMaxRowsPerSplit;
    pl.rows_per_split = rows;
    pl.k_splits = (Z + rows - 1) / rows;
    // The arrival counters sit in a fixed-size area in front of the partial sums, whatever the shape: a
    // workspace shared by launches of different shapes (the projections of a decode step) must never have
    // one shape's partial sums land on another shape's counters.
    pl.counter_bytes = round_up(sizeof(int) * (size_t)pl.n_slices, kCounterAreaBytes);
    pl.partial_bytes =
        pl.k_splits > 1 ? sizeof(float) * (size_t)pl.k_splits * arrays * pl.n_slices * kColsPerCta : 0;
    return pl;
}

__device__ __forceinline__ void fma8(float (&acc)[8], const uint4& w, float xv) {
    float2 a = h2_to_f2(w.x), b = h2_to_f2(w.y), c = h2_to_f2(w.z), d = h2_to_f2(w.w);
    acc[0] = fmaf(a.x, xv, acc[0]);
    acc[1] = fmaf(a.y, xv, acc[1]);
    acc[2] = fmaf(b.x, xv, acc[2]);
    acc[3] = fmaf(b.y, xv, acc[3]);
    acc[4] = fmaf(c.x, xv, acc[4]);
    acc[5] = fmaf(c.y, xv, acc[5]);
    acc[6] = fmaf(d.x, xv, acc[6]);
    acc[7] = fmaf(d.y, xv, acc[7]);
}

template <bool kSwiglu>
__global__ void __launch_bounds__(kThreads, kSwiglu ? 3 : 4) sparse_gemv_kernel(const GemvParams p) {
    constexpr int kArrays = kSwiglu ? 2 : 1;
    constexpr int kUnroll = kSwiglu ? 4 : 8;

    __shared__ uint16_t s_row[kMaxRowsPerSplit];
    __shared__ float s_x[kMaxRowsPerSplit];
    __shared__ float s_x2[kSwiglu ? kMaxRowsPerSplit : 1];
    __shared__ __align__(16) float s_red[kWarps][kArrays][kColsPerCta];
    __shared__ int s_wcount[kWarps];
    __shared__ int s_last;

    // The weights are constants, not an output of the previous kernel: the first rows of this CTA's range are
    // asked into L2 before the dependency wait, so that they arrive while the previous kernel drains and while
    // this CTA tests and compacts its input channels. Which rows are active is not known yet, so about
    // (sparsity) of these bytes are not used; the count is kept small.
    if (p.prefetch_rows > 0) {
        const int z0p = blockIdx.y * p.rows_per_split;
        const int nr = min(p.prefetch_rows, min(p.rows_per_split, p.Z - z0p));
        const int colb = blockIdx.x * kColsPerCta;
        const int bytes = min(kColsPerCta, p.N - colb) * 2;           // N % 8 == 0: a multiple of 16
        const int t = threadIdx.x;
        if (t < nr * kArrays && bytes > 0) {
            const int r = kSwiglu ? t >> 1 : t;
            const __half* base = (kSwiglu && (t & 1)) ? p.Wt2 : p.Wt;
            const __half* a = base + (size_t)(z0p + r) * p.N + colb;
            asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(a), "r"(bytes) : "memory");
        }
    }
    pdl_begin();
    const int tid = threadIdx.x;
    const int warp = tid >> 5, lane = tid & 31;
    const int slice = blockIdx.x;
    const int z0 = blockIdx.y * p.rows_per_split;
    const int nrows = min(p.rows_per_split, p.Z - z0);

    // Fused RMSNorm: every CTA derives the row's scale itself (Z * 2 bytes from L2, a few hundred
    // FMAs) instead of waiting for a separate one-CTA kernel. The summation order is the same in
    // every CTA, so all of them see the same x.
    float rnorm = 0.f;
    // rows this lane will test during compaction: start their loads now, they overlap the norm's reduction
    const int per_warp = (nrows + kWarps - 1) / kWarps;
    const int w0 = warp * per_warp;
    const int w1 = min(nrows, w0 + per_warp);
    __half xraw[kLaneSlots], nw[kLaneSlots];
#pragma unroll
    for (int s = 0; s < kLaneSlots; ++s) {
        const int r = w0 + s * 32 + lane;
        xraw[s] = r < w1 ? p.x[z0 + r] : __float2half_rn(0.f);
        nw[s] = (r < w1 && p.norm_w != nullptr) ? p.norm_w[z0 + r] : __float2half_rn(0.f);
    }
    if (p.norm_w != nullptr) {
        float ss = 0.f;
        const uint4* hv = reinterpret_cast<const uint4*>(p.x);
#pragma unroll 4
        for (int i = tid; i < (p.Z >> 3); i += kThreads) {
            const uint4 a = hv[i];
            const float2 f0 = h2_to_f2(a.x), f1 = h2_to_f2(a.y), f2 = h2_to_f2(a.z), f3 = h2_to_f2(a.w);
            ss = fmaf(f0.x, f0.x, ss); ss = fmaf(f0.y, f0.y, ss);
            ss = fmaf(f1.x, f1.x, ss); ss = fmaf(f1.y, f1.y, ss);
            ss = fmaf(f2.x, f2.x, ss); ss = fmaf(f2.y, f2.y, ss);
            ss = fmaf(f3.x, f3.x, ss); ss = fmaf(f3.y, f3.y, ss);
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        if (lane == 0) s_red[0][0][warp] = ss;
        __syncthreads();
        float tot = 0.f;
#pragma unroll
        for (int w = 0; w < kWarps; ++w) tot += s_red[0][0][w];
        rnorm = rsqrtf(tot / (float)p.Z + p.norm_eps);
        __syncthreads();   // s_red is reused below
    }

    // Threshold of the projection this column slice belongs to.
    float thr = p.thr[0];
    if (!kSwiglu) {
        const int c = slice * kColsPerCta;
        int s = 0;
        while (s + 1 < p.n_segments && c >= p.seg_end[s]) ++s;
        thr = p.thr[s];
    }
    const __half thr_h = __float2half_rn(thr);
    const __half thr2_h = __float2half_rn(kSwiglu ? p.thr_up : thr);

    // ---- threshold test + ordered compaction of this CTA's input channels ----
    float xv[kLaneSlots], xv2[kLaneSlots];
    int pos[kLaneSlots];
    bool act[kLaneSlots];
    int wtotal = 0;
#pragma unroll
    for (int s = 0; s < kLaneSlots; ++s) {
        const int r = w0 + s * 32 + lane;
        bool a = false;
        float v = 0.f, v2 = 0.f;
        if (r < w1) {
            __half h = xraw[s];
            if (p.norm_w != nullptr) h = __hmul(nw[s], __float2half_rn(__half2float(h) * rnorm));
            const __half m = __habs(h);
            const bool a1 = __hgt(m, thr_h);
            const bool a2 = kSwiglu ? __hgt(m, thr2_h) : a1;
            a = a1 || a2;
            const float f = __half2float(h);
            v = a1 ? f : 0.f;
            v2 = a2 ? f : 0.f;
        }
        const unsigned b = __ballot_sync(0xffffffffu, a);
        pos[s] = wtotal + __popc(b & ((1u << lane) - 1u));
        act[s] = a;
        xv[s] = v;
        xv2[s] = v2;
        wtotal += __popc(b);
    }
    if (lane == 0) s_wcount[warp] = wtotal;
    __syncthreads();
    int base = 0, total = 0;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) {
        const int c = s_wcount[w];
        if (w < warp) base += c;
        total += c;
    }
#pragma unroll
    for (int s = 0; s < kLaneSlots; ++s) {
        if (act[s]) {
            const int e = base + pos[s];
            s_row[e] = (uint16_t)(w0 + s * 32 + lane);
            s_x[e] = xv[s];
            if (kSwiglu) s_x2[e] = xv2[s];
        }
    }
    __syncthreads();

    // ---- stream the active weight rows ----
    const int col0 = slice * kColsPerCta + lane * 8;
    const bool col_ok = col0 < p.N;   // N % 8 == 0: a lane's 8 columns are all in or all out
    const size_t ldw = (size_t)p.N;
    const __half* wbase = p.Wt + (size_t)z0 * ldw + col0;
    const __half* wbase2 = kSwiglu ? p.Wt2 + (size_t)z0 * ldw + col0 : nullptr;

    float acc[8], acc2[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = acc2[j] = 0.f;

    if (col_ok) {
        for (int e0 = warp; e0 < total; e0 += kWarps * kUnroll) {
            uint4 w[kUnroll], w2[kSwiglu ? kUnroll : 1];
            float xs[kUnroll], xs2[kSwiglu ? kUnroll : 1];
#pragma unroll
            for (int u = 0; u < kUnroll; ++u) {
                const int e = e0 + u * kWarps;
                if (e < total) {
                    const size_t off = (size_t)s_row[e] * ldw;
                    w[u] = ld_stream_16(wbase + off);
                    xs[u] = s_x[e];
                    if (kSwiglu) {
                        w2[u] = ld_stream_16(wbase2 + off);
                        xs2[u] = s_x2[e];
                    }
                } else {
                    w[u] = make_uint4(0, 0, 0, 0);
                    xs[u] = 0.f;
                    if (kSwiglu) {
                        w2[u] = make_uint4(0, 0, 0, 0);
                        xs2[u] = 0.f;
                    }
                }
            }
#pragma unroll
            for (int u = 0; u < kUnroll; ++u) {
                fma8(acc, w[u], xs[u]);
                if (kSwiglu) fma8(acc2, w2[u], xs2[u]);
            }
        }
    }

    // ---- CTA reduction over the 8 warps (fixed order) ----
    {
        float4* d = reinterpret_cast<float4*>(&s_red[warp][0][lane * 8]);
        d[0] = make_float4(acc[0], acc[1], acc[2], acc[3]);
        d[1] = make_float4(acc[4], acc[5], acc[6], acc[7]);
        if (kSwiglu) {
            float4* d2 = reinterpret_cast<float4*>(&s_red[warp][kArrays - 1][lane * 8]);
            d2[0] = make_float4(acc2[0], acc2[1], acc2[2], acc2[3]);
            d2[1] = make_float4(acc2[4], acc2[5], acc2[6], acc2[7]);
        }
    }
    __syncthreads();
    float sum = 0.f, sum2 = 0.f;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) {
        sum += s_red[w][0][tid];
        if (kSwiglu) sum2 += s_red[w][kArrays - 1][tid];
    }

    const int col = slice * kColsPerCta + tid;
    const int npad = p.n_slices * kColsPerCta;

    if (p.active_elems != nullptr && tid == 0) {
        const int cols_here = min(kColsPerCta, p.N - slice * kColsPerCta);
        atomicAdd(p.active_elems, (unsigned long long)total * cols_here * kArrays);
    }

    if (p.k_splits > 1) {
        float* mine = p.partials + ((size_t)blockIdx.y * kArrays) * npad + col;
        mine[0] = sum;
        if (kSwiglu) mine[npad] = sum2;
        __threadfence();
        __syncthreads();
        if (tid == 0) {
            const int prev = atomicAdd(&p.counters[slice], 1);
            s_last = (prev == p.k_splits - 1);
        }
        __syncthreads();
        if (!s_last) return;
        __threadfence();
        // Final merge, spread over the whole CTA so that it costs a couple of L2 round trips
        // instead of k_splits: warp w sums splits w, w+8, ... (ascending) for all 256 columns,
        // then the 8 warp sums are added in warp order. The order is fixed, so the result is too.
        {
            float m[8], m2[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) m[j] = m2[j] = 0.f;
            const float* base = p.partials + slice * kColsPerCta + lane * 8;
            // kBatch splits' loads are issued together (one L2 round trip for up to 8 * kBatch splits);
            // the sums are still taken in ascending split order
            constexpr int kBatch = kSwiglu ? 2 : 5;
            for (int k0 = warp; k0 < p.k_splits; k0 += kWarps * kBatch) {
                float4 a[kBatch], b[kBatch], c[kSwiglu ? kBatch : 1], d[kSwiglu ? kBatch : 1];
#pragma unroll
                for (int i = 0; i < kBatch; ++i) {
                    const int k = k0 + i * kWarps;
                    const float* src = base + ((size_t)k * kArrays) * npad;
                    const bool ok = k < p.k_splits;
                    a[i] = ok ? ld_cg_f32x4(src) : make_float4(0.f, 0.f, 0.f, 0.f);
                    b[i] = ok ? ld_cg_f32x4(src + 4) : make_float4(0.f, 0.f, 0.f, 0.f);
                    if (kSwiglu) {
                        c[i] = ok ? ld_cg_f32x4(src + npad) : make_float4(0.f, 0.f, 0.f, 0.f);
                        d[i] = ok ? ld_cg_f32x4(src + npad + 4) : make_float4(0.f, 0.f, 0.f, 0.f);
                    }
                }
#pragma unroll
                for (int i = 0; i < kBatch; ++i) {
                    if (k0 + i * kWarps < p.k_splits) {
                        m[0] += a[i].x; m[1] += a[i].y; m[2] += a[i].z; m[3] += a[i].w;
                        m[4] += b[i].x; m[5] += b[i].y; m[6] += b[i].z; m[7] += b[i].w;
                        if (kSwiglu) {
                            m2[0] += c[i].x; m2[1] += c[i].y; m2[2] += c[i].z; m2[3] += c[i].w;
                            m2[4] += d[i].x; m2[5] += d[i].y; m2[6] += d[i].z; m2[7] += d[i].w;
                        }
                    }
                }
            }
            float4* d = reinterpret_cast<float4*>(&s_red[warp][0][lane * 8]);
            d[0] = make_float4(m[0], m[1], m[2], m[3]);
            d[1] = make_float4(m[4], m[5], m[6], m[7]);
            if (kSwiglu) {
                float4* d2 = reinterpret_cast<float4*>(&s_red[warp][kArrays - 1][lane * 8]);
                d2[0] = make_float4(m2[0], m2[1], m2[2], m2[3]);
                d2[1] = make_float4(m2[4], m2[5], m2[6], m2[7]);
            }
        }
        __syncthreads();
        sum = 0.f;
        sum2 = 0.f;
#pragma unroll
        for (int w = 0; w < kWarps; ++w) {
            sum += s_red[w][0][tid];
            if (kSwiglu) sum2 += s_red[w][kArrays - 1][tid];
        }
        if (tid == 0) p.counters[slice] = 0;   // leave the workspace ready for the next launch
    }

    if (!kSwiglu && p.xw > 0) {
        // Sum of the ranks' partial products, inside this kernel: every thread of the CTA that holds
        // a finished 256-column tile sends its column's fp32 value, tagged with the step's epoch, to
        // every rank's receive area (one 64-bit store each, NVLink for the peers), then polls its
        // column's words here until each carries this epoch, and adds them in rank order, so every
        // rank ends up with the same bits. Epochs only grow, so nothing is ever reset. A poll that
        // runs out sets the status word, which also turns all later polls off (the result is then
        // meaningless, but no kernel hangs).
        const unsigned int ep = (unsigned int)*reinterpret_cast<const volatile int*>(p.xepoch);
        const unsigned long long word = ((unsigned long long)ep << 32) | (unsigned long long)__float_as_uint(sum);
        // every rank starts with a different destination so that the ranks' stores do not all converge on
        // one GPU's links at the same moment
        for (int i = 0; i < p.xw; ++i) {
            int r = p.xrank + i;
            r = r >= p.xw ? r - p.xw : r;
            st_relaxed_sys_u64(p.xrecv[r] + (size_t)p.xrank * npad + col, word);
        }
        const bool live = *reinterpret_cast<volatile int*>(p.xstatus) == 0;
        // first look at every source at once (independent loads), then poll whatever is still missing
        unsigned long long v[LEANKV_MAX_RANKS];
        const unsigned long long* src0 = p.xrecv[p.xrank] + col;
#pragma unroll
        for (int r = 0; r < LEANKV_MAX_RANKS; ++r)
            v[r] = r < p.xw ? ld_relaxed_sys_u64(src0 + (size_t)r * npad) : 0ull;
        float tot = 0.f;
        bool ok = live;
#pragma unroll
        for (int r = 0; r < LEANKV_MAX_RANKS; ++r) {
            if (r < p.xw) {
                if (live) {
                    int it = 0;
                    while ((unsigned int)(v[r] >> 32) != ep && it < p.xlimit) {
                        __nanosleep(20);
                        v[r] = ld_relaxed_sys_u64(src0 + (size_t)r * npad);
                        ++it;
                    }
                    ok = ok && (unsigned int)(v[r] >> 32) == ep;
                }
                tot += __uint_as_float((unsigned int)v[r]);
            }
        }
        if (!ok && live) atomicOr(p.xstatus, 1);
        sum = tot;
    }

    if (col >= p.N) return;
    if (kSwiglu) {
        // Rounding points of the two-GEMV + act_fn(gate)*up path: fp16 gate, fp16 up,
        // silu evaluated in fp32 and rounded, fp16 product.
        const __half g16 = __float2half_rn(sum);
        const __half u16 = __float2half_rn(sum2);
        const float gf = __half2float(g16);
        const __half s16 = __float2half_rn(gf / (1.0f + expf(-gf)));
        p.y[col] = __hmul(s16, u16);
    } else {
        __half r = __float2half_rn(sum);
        if (p.bias != nullptr) r = __hadd(r, p.bias[col]);
        if (p.residual != nullptr) r = __hadd(p.residual[col], r);
        p.y[col] = r;
    }
}

int check_common(const void* Wt, const void* x, const void* y, int N, int Z) {
    if (Wt == nullptr || x == nullptr || y == nullptr) return LEANKV_EINVAL;
    if (N <= 0 || Z <= 0) return LEANKV_EINVAL;
    if (N % 8 != 0) return LEANKV_EALIGN;
    if (!aligned16(Wt) || !aligned16(y)) return LEANKV_EALIGN;
    if ((reinterpret_cast<uintptr_t>(x) & 1u) != 0) return LEANKV_EALIGN;
    return LEANKV_OK;
}

// With the RMSNorm fused in, every CTA reads the whole input row for the norm while the finishing CTAs
// of other column slices are already writing y: the output must not overlap the input row.
int check_norm(const void* x, const void* norm_w, int Z, const void* y, int N) {
    if (norm_w == nullptr) return LEANKV_OK;
    if (Z % 8 != 0 || !aligned16(x) || (reinterpret_cast<uintptr_t>(norm_w) & 1u) != 0) return LEANKV_EALIGN;
    const uintptr_t x0 = reinterpret_cast<uintptr_t>(x), x1 = x0 + 2 * (uintptr_t)Z;
    const uintptr_t y0 = reinterpret_cast<uintptr_t>(y), y1 = y0 + 2 * (uintptr_t)N;
    if (y0 < x1 && x0 < y1) return LEANKV_EINVAL;
    return LEANKV_OK;
}

int launch_gemv(const void* Wt, const void* x, void* y, int N, int Z, const leankv_segments_t* segs,
                const void* bias, const void* residual, void* workspace, size_t workspace_bytes,
                unsigned long long* active, void* stream, const void* norm_w = nullptr, float norm_eps = 0.f,
                const leankv_xchg_t* xchg = nullptr, int slot = 0) {
    int rc = check_common(Wt, x, y, N, Z);
    if (rc != LEANKV_OK) return rc;
    rc = check_norm(x, norm_w, Z, y, N);
    if (rc != LEANKV_OK) return rc;
    if (segs == nullptr || segs->n_segments < 1 || segs->n_segments > LEANKV_MAX_SEGMENTS)
        return LEANKV_EINVAL;
    int prev = 0;
    for (int s = 0; s < segs->n_segments; ++s) {
        const int e = segs->seg_end[s];
        if (e <= prev) return LEANKV_EINVAL;
        if (s + 1 < segs->n_segments && e % kColsPerCta != 0) return LEANKV_EALIGN;
        prev = e;
    }
    if (prev != N) return LEANKV_EINVAL;

    const GemvPlan pl = make_plan(N, Z, 1);
    if (pl.k_splits > 1) {
        if (workspace == nullptr || workspace_bytes < pl.counter_bytes + pl.partial_bytes)
            return LEANKV_EWORKSPACE;
        if (!aligned16(workspace)) return LEANKV_EALIGN;
    }
    GemvParams p{};
    p.Wt = static_cast<const __half*>(Wt);
    p.Wt2 = nullptr;
    p.x = static_cast<const __half*>(x);
    p.y = static_cast<__half*>(y);
    p.bias = static_cast<const __half*>(bias);
    p.residual = static_cast<const __half*>(residual);
    p.counters = static_cast<int*>(workspace);
    p.partials = reinterpret_cast<float*>(static_cast<char*>(workspace) + pl.counter_bytes);
    p.active_elems = active;
    p.N = N;
    p.Z = Z;
    p.n_slices = pl.n_slices;
    p.k_splits = pl.k_splits;
    p.rows_per_split = pl.rows_per_split;
    p.prefetch_rows = prefetch_rows(pl.rows_per_split, 1);
    p.n_segments = segs->n_segments;
    for (int s = 0; s < LEANKV_MAX_SEGMENTS; ++s) {
        p.seg_end[s] = s < segs->n_segments ? segs->seg_end[s] : N;
        p.thr[s] = s < segs->n_segments ? segs->threshold[s] : 0.f;
    }
    p.thr_up = 0.f;
    p.norm_w = static_cast<const __half*>(norm_w);
    p.norm_eps = norm_eps;
    if (xchg != nullptr) {
        const int npad = pl.n_slices * kColsPerCta;
        if (xchg->world < 1 || xchg->world > LEANKV_MAX_RANKS || xchg->rank < 0 || xchg->rank >= xchg->world ||
            slot < 0 || slot >= xchg->n_slots || npad > xchg->max_cols || !xchg->epoch || !xchg->status ||
            xchg->max_wait_iters < 1)
            return LEANKV_EINVAL;
        p.xw = xchg->world;
        p.xrank = xchg->rank;
        p.xlimit = xchg->max_wait_iters;
        p.xepoch = xchg->epoch;
        p.xstatus = xchg->status;
        for (int r = 0; r < xchg->world; ++r) {
            if (!xchg->recv[r] || (reinterpret_cast<uintptr_t>(xchg->recv[r]) & 7u) != 0) return LEANKV_EINVAL;
            p.xrecv[r] = static_cast<unsigned long long*>(xchg->recv[r]) +
                         (size_t)slot * xchg->world * xchg->max_cols;
        }
    }
    dim3 grid(pl.n_slices, pl.k_splits);
    LEANKV_CUDA_TRY(launch_kernel_ex(true, sparse_gemv_kernel<false>, grid, dim3(kThreads), 0,
                                  static_cast<cudaStream_t>(stream), p));
    return LEANKV_OK;
}

}  // namespace
}  // namespace leankv

using namespace leankv;

extern "C" size_t leankv_sparse_gemv_workspace_bytes(int N, int Z) {
    if (N <= 0 || Z <= 0) return 0;
    const GemvPlan pl = make_plan(N, Z, 1);
    return pl.counter_bytes + pl.partial_bytes;
}

extern "C" size_t leankv_sparse_swiglu_workspace_bytes(int N, int Z) {
    if (N <= 0 || Z <= 0) return 0;
    const GemvPlan pl = make_plan(N, Z, 2);
    return pl.counter_bytes + pl.partial_bytes;
}

extern "C" int leankv_sparse_gemv_f16(const void* Wt, const void* x, void* y, int N, int Z,
                                      float threshold, const void* bias, const void* residual,
                                      void* workspace, size_t workspace_bytes,
                                      unsigned long long* active_elems, void* stream) {
    leankv_segments_t segs{};
    segs.n_segments = 1;
    segs.seg_end[0] = N;
    segs.threshold[0] = threshold;
    return launch_gemv(Wt, x, y, N, Z, &segs, bias, residual, workspace, workspace_bytes,
                       active_elems, stream);
}

extern "C" int leankv_sparse_gemv_seg_f16(const void* Wt, const void* x, void* y, int N, int Z,
                                          const leankv_segments_t* segs, const void* bias,
                                          const void* residual, void* workspace,
                                          size_t workspace_bytes, unsigned long long* active_elems,
                                          void* stream) {
    return launch_gemv(Wt, x, y, N, Z, segs, bias, residual, workspace, workspace_bytes,
                       active_elems, stream);
}

extern "C" size_t leankv_xchg_recv_bytes(int world, int n_slots, int max_cols) {
    if (world < 1 || n_slots < 1 || max_cols < 1) return 0;
    return sizeof(unsigned long long) * (size_t)n_slots * world * max_cols;
}

static __global__ void xchg_advance_kernel(int* epoch) {
    pdl_begin();
    *epoch = *epoch + 1;
}

extern "C" int leankv_xchg_advance(int32_t* epoch, void* stream) {
    if (!epoch) return LEANKV_EINVAL;
    LEANKV_CUDA_TRY(launch_kernel(xchg_advance_kernel, dim3(1), dim3(1), 0, static_cast<cudaStream_t>(stream), epoch));
    return LEANKV_OK;
}

extern "C" int leankv_sparse_gemv_allreduce_f16(const void* Wt, const void* x, void* y, int N, int Z,
                                                float threshold, const void* residual, void* workspace,
                                                size_t workspace_bytes, unsigned long long* active_elems,
                                                const leankv_xchg_t* xchg, int slot, void* stream) {
    if (!xchg || xchg->max_cols % kColsPerCta != 0) return LEANKV_EINVAL;
    leankv_segments_t segs{};
    segs.n_segments = 1;
    segs.seg_end[0] = N;
    segs.threshold[0] = threshold;
    return launch_gemv(Wt, x, y, N, Z, &segs, nullptr, residual, workspace, workspace_bytes, active_elems,
                       stream, nullptr, 0.f, xchg, slot);
}

static int launch_swiglu(const void* Wt_gate, const void* Wt_up, const void* x, void* y, int N, int Z,
                         float t_gate, float t_up, void* workspace, size_t workspace_bytes,
                         unsigned long long* active_elems, void* stream, const void* norm_w, float norm_eps) {
    int rc = check_common(Wt_gate, x, y, N, Z);
    if (rc != LEANKV_OK) return rc;
    rc = check_norm(x, norm_w, Z, y, N);
    if (rc != LEANKV_OK) return rc;
    if (Wt_up == nullptr) return LEANKV_EINVAL;
    if (!aligned16(Wt_up)) return LEANKV_EALIGN;
    const GemvPlan pl = make_plan(N, Z, 2);
    if (pl.k_splits > 1) {
        if (workspace == nullptr || workspace_bytes < pl.counter_bytes + pl.partial_bytes)
            return LEANKV_EWORKSPACE;
        if (!aligned16(workspace)) return LEANKV_EALIGN;
    }
    GemvParams p{};
    p.Wt = static_cast<const __half*>(Wt_gate);
    p.Wt2 = static_cast<const __half*>(Wt_up);
    p.x = static_cast<const __half*>(x);
    p.y = static_cast<__half*>(y);
    p.counters = static_cast<int*>(workspace);
    p.partials = reinterpret_cast<float*>(static_cast<char*>(workspace) + pl.counter_bytes);
    p.active_elems = active_elems;
    p.N = N;
    p.Z = Z;
    p.n_slices = pl.n_slices;
    p.k_splits = pl.k_splits;
    p.rows_per_split = pl.rows_per_split;
    p.prefetch_rows = prefetch_rows(pl.rows_per_split, 2);
    p.n_segments = 1;
    for (int s = 0; s < LEANKV_MAX_SEGMENTS; ++s) {
        p.seg_end[s] = N;
        p.thr[s] = t_gate;
    }
    p.thr_up = t_up;
    p.norm_w = static_cast<const __half*>(norm_w);
    p.norm_eps = norm_eps;
    dim3 grid(pl.n_slices, pl.k_splits);
    LEANKV_CUDA_TRY(launch_kernel_ex(true, sparse_gemv_kernel<true>, grid, dim3(kThreads), 0,
                                  static_cast<cudaStream_t>(stream), p));
    return LEANKV_OK;
}

extern "C" int leankv_sparse_swiglu_f16(const void* Wt_gate, const void* Wt_up, const void* x,
                                        void* y, int N, int Z, float t_gate, float t_up,
                                        void* workspace, size_t workspace_bytes,
                                        unsigned long long* active_elems, void* stream) {
    return launch_swiglu(Wt_gate, Wt_up, x, y, N, Z, t_gate, t_up, workspace, workspace_bytes, active_elems,
                         stream, nullptr, 0.f);
}

extern "C" int leankv_sparse_gemv_rmsnorm_f16(const void* Wt, const void* h, const void* norm_weight,
                                              float eps, void* y, int N, int Z,
                                              const leankv_segments_t* segs, const void* residual,
                                              void* workspace, size_t workspace_bytes,
                                              unsigned long long* active_elems, void* stream) {
    if (norm_weight == nullptr) return LEANKV_EINVAL;
    return launch_gemv(Wt, h, y, N, Z, segs, nullptr, residual, workspace, workspace_bytes, active_elems,
                       stream, norm_weight, eps);
}

extern "C" int leankv_sparse_swiglu_rmsnorm_f16(const void* Wt_gate, const void* Wt_up, const void* h,
                                                const void* norm_weight, float eps, void* y, int N, int Z,
                                                float t_gate, float t_up, void* workspace,
                                                size_t workspace_bytes, unsigned long long* active_elems,
                                                void* stream) {
    if (norm_weight == nullptr) return LEANKV_EINVAL;
    return launch_swiglu(Wt_gate, Wt_up, h, y, N, Z, t_gate, t_up, workspace, workspace_bytes, active_elems,
                         stream, norm_weight, eps);
}

// ---------------------------------------------------------------------------------------------
// Sparse GEMV for callers that may not allocate device memory.
//
// Some hosts of this library cannot hand over a workspace: a serving process whose memory pool
// has already claimed the whole GPU (any further cudaMalloc fails or stalls the device), a plugin
// sandbox in which only the host application may call the allocator, or a latency-critical loop
// where an allocation's implicit device synchronisation is not acceptable. For them the split-K
// scratch lives in the library image itself: a fixed array in device global memory that every GPU
// loading the library carries until the process exits.
// ---------------------------------------------------------------------------------------------
namespace leankv {
namespace {

constexpr size_t kStaticScratchBytes = 768u << 10;   // 768 KiB per GPU, resident for the process lifetime
constexpr int kStaticMaxDim = 65536;                 // largest N or Z this entry point accepts
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

// Device address of g_static_scratch per device ordinal. In host code the symbol's name is only a
// handle for the runtime, never a pointer a kernel could use; the address has to be asked for.
// The table is filled without a lock: threads that race on a device's first call all store the same
// address (a pointer-sized store), so the worst case is a repeated look-up.
constexpr int kStaticMaxDevices = 64;
void* g_static_scratch_addr[kStaticMaxDevices] = {nullptr};

}  // namespace
}  // namespace leankv

extern "C" int leankv_sparse_gemv_f16_static(const void* Wt, const void* x, void* y, int N, int Z,
                                             float threshold, void* stream) {
    int rc = check_common(Wt, x, y, N, Z);
    if (rc != LEANKV_OK) return rc;
    if (N > kStaticMaxDim || Z > kStaticMaxDim) return LEANKV_ELIMIT;
    const GemvPlan pl = make_plan(N, Z, 1);
    if (pl.counter_bytes + pl.partial_bytes > kStaticScratchBytes) return LEANKV_ELIMIT;

    int dev = 0;
    LEANKV_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= kStaticMaxDevices) return LEANKV_ELIMIT;
    if (g_static_scratch_addr[dev] == nullptr) {
        // One-time set-up for this device (it must be the current device, which it is). This may
        // load the module, so the first call on a device belongs before any stream capture.
        void* addr = nullptr;
        LEANKV_CUDA_TRY(cudaGetSymbolAddress(&addr, g_static_scratch));
        g_static_scratch_addr[dev] = addr;
    }
    void* scratch = g_static_scratch_addr[dev];
    // The array keeps whatever the previous call left. Only the arrival counters must start at zero
    // (partials are fully overwritten before they are read), so those are cleared on the stream.
    if (pl.k_splits > 1)
        LEANKV_CUDA_TRY(cudaMemsetAsync(scratch, 0, pl.counter_bytes, static_cast<cudaStream_t>(stream)));

    leankv_segments_t segs{};
    segs.n_segments = 1;
    segs.seg_end[0] = N;
    segs.threshold[0] = threshold;
    return launch_gemv(Wt, x, y, N, Z, &segs, nullptr, nullptr, scratch, kStaticScratchBytes, nullptr, stream);
}
