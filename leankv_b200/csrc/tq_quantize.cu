// TurboQuant (MSE variant) quantize / dequantize and the paged-pool append for B200.
//
// Arithmetic contract shared by every kernel in this file (and restated on the CPU by
// the test oracle), chosen so that a vector's codes never depend on how vectors are
// batched, tiled or appended:
//   norm   = float( sqrt( S_lo + S_hi ) ),  S_lo / S_hi = fp64 sums of squares of
//            coordinates 0..63 / 64..127 taken in ascending order
//   u[k]   = x[k] / (norm + 1e-10f)                       (fp32, IEEE division)
//   y[j]   = fma(Pi[j][127], u[127], ... fma(Pi[j][0], u[0], 0))   (fp32, ascending k)
//   code_j = #{ i : boundary[i] < y[j] }
// This is leankv/turboquant/quantizer.py:119-129; the reference leaves the summation
// order to its BLAS, so a code can differ from it only where y lies within rounding
// distance of a decision boundary.

#include <cstdlib>

#include "common.cuh"
#include "tq_layout.cuh"
#include "umma.cuh"

namespace leankv {
namespace {

constexpr int kDim = LEANKV_TQ_DIM;
constexpr int kTileVecs = 128;
constexpr int kTileThreads = 256;
constexpr size_t kTileSmemBytes = 2 * (size_t)kDim * 128 * sizeof(float);   // A and B panels

__device__ __forceinline__ int packed_len_dev(int bits) {
    return bits == 1 ? kDim / 8 : bits == 2 ? kDim / 4 : bits <= 4 ? kDim / 2 : kDim;
}

// Sum of squares of 64 values in fp64, ascending order.
__device__ __forceinline__ double sumsq64(const float (&x)[64]) {
    double s = 0.0;
#pragma unroll
    for (int i = 0; i < 64; ++i) s = fma((double)x[i], (double)x[i], s);
    return s;
}

struct TileParams {
    const void* x;          // quantize: input vectors; dequantize: unused
    int x_dtype;            // 0 fp16, 1 fp32
    long long n_vec;
    int bits;
    const float* Pi;
    const float* table;     // quantize: decision boundaries (2^bits-1); dequantize: centroids
    uint8_t* indices;
    float* norms;
    void* out;              // dequantize output
    int out_dtype;
};

// One CTA = 128 vectors x 128 coordinates, 8x8 register tile per thread, k ascending.
// kQuantize: A[k][v] = u_v[k], B[k][j] = Pi[j][k]  -> y ; else A[k][v] = c[code_v[k]],
// B[k][j] = Pi[k][j] -> x_hat (rotate_backward, leankv/turboquant/rotation.py:50-52).
template <bool kQuantize>
__global__ void __launch_bounds__(kTileThreads, 1) tq_tile_kernel(const TileParams p) {
    extern __shared__ __align__(16) float smem[];
    float* s_a = smem;                 // [k][128 vectors]
    float* s_b = smem + kDim * 128;    // [k][128 coords]
    __shared__ float s_norm[kTileVecs];
    __shared__ float s_table[16];

    const int tid = threadIdx.x;
    const int bits = p.bits;
    const int n_table = kQuantize ? (1 << bits) - 1 : (1 << bits);
    if (tid < 16) s_table[tid] = tid < n_table ? p.table[tid] : __int_as_float(0x7f800000);

    // B panel, loaded once per CTA (persistent over tiles).
    for (int i = tid; i < kDim * kDim; i += kTileThreads) {
        if (kQuantize) {
            const int j = i & 127, k = i >> 7;   // lanes walk j: strided global read, conflict-free store
            s_b[k * 128 + j] = p.Pi[j * kDim + k];
        } else {
            s_b[i] = p.Pi[i];
        }
    }

    const int plen = packed_len_dev(bits);
    const int vpb = kDim / plen;                  // codes per byte
    const int bw = 8 / vpb;                       // bits per packed field
    const long long n_tiles = (p.n_vec + kTileVecs - 1) / kTileVecs;

    for (long long tile = blockIdx.x; tile < n_tiles; tile += gridDim.x) {
        const long long v0 = tile * kTileVecs;
        __syncthreads();   // previous tile's readers of s_a are done; tables are visible
        {
            const int v = tid >> 1, hf = tid & 1;
            const long long gv = v0 + v;
            const bool ok = gv < p.n_vec;
            if (kQuantize) {
                float xr[64];
                if (ok && p.x_dtype == 0) {
                    const uint4* src = reinterpret_cast<const uint4*>(
                        static_cast<const __half*>(p.x) + gv * kDim + hf * 64);
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        const uint4 w = __ldg(src + i);
                        const float2 a = h2_to_f2(w.x), b = h2_to_f2(w.y), c = h2_to_f2(w.z),
                                     d = h2_to_f2(w.w);
                        xr[8 * i + 0] = a.x; xr[8 * i + 1] = a.y; xr[8 * i + 2] = b.x; xr[8 * i + 3] = b.y;
                        xr[8 * i + 4] = c.x; xr[8 * i + 5] = c.y; xr[8 * i + 6] = d.x; xr[8 * i + 7] = d.y;
                    }
                } else if (ok) {
                    const float4* src = reinterpret_cast<const float4*>(
                        static_cast<const float*>(p.x) + gv * kDim + hf * 64);
#pragma unroll
                    for (int i = 0; i < 16; ++i) {
                        const float4 w = __ldg(src + i);
                        xr[4 * i + 0] = w.x; xr[4 * i + 1] = w.y; xr[4 * i + 2] = w.z; xr[4 * i + 3] = w.w;
                    }
                } else {
#pragma unroll
                    for (int i = 0; i < 64; ++i) xr[i] = 0.f;
                }
                const double mine = sumsq64(xr);
                const double other = __shfl_xor_sync(0xffffffffu, mine, 1);
                const double tot = hf == 0 ? mine + other : other + mine;
                const float norm = (float)sqrt(tot);
                const float denom = norm + 1e-10f;
                if (hf == 0) s_norm[v] = norm;
#pragma unroll
                for (int i = 0; i < 64; ++i) s_a[(hf * 64 + i) * 128 + v] = xr[i] / denom;
            } else {
                const uint32_t mask = (1u << bw) - 1u;
                const int bytes_half = plen / 2;
                const uint8_t* src = p.indices + gv * plen + hf * bytes_half;
                for (int bi = 0; bi < bytes_half; ++bi) {
                    const uint32_t byte = ok ? src[bi] : 0u;
                    for (int q = 0; q < vpb; ++q) {
                        const int k = hf * 64 + bi * vpb + q;
                        const int code = (byte >> (q * bw)) & mask;
                        s_a[k * 128 + v] = ok ? s_table[code & 15] : 0.f;
                    }
                }
                if (hf == 0) s_norm[v] = ok ? p.norms[gv] : 0.f;
            }
        }
        __syncthreads();

        const int tm = tid >> 4, tn = tid & 15;
        float acc[8][8];
#pragma unroll
        for (int i = 0; i < 8; ++i)
#pragma unroll
            for (int j = 0; j < 8; ++j) acc[i][j] = 0.f;

#pragma unroll 4
        for (int k = 0; k < kDim; ++k) {
            const float4 a0 = *reinterpret_cast<const float4*>(&s_a[k * 128 + tm * 8]);
            const float4 a1 = *reinterpret_cast<const float4*>(&s_a[k * 128 + tm * 8 + 4]);
            const float4 b0 = *reinterpret_cast<const float4*>(&s_b[k * 128 + tn * 4]);
            const float4 b1 = *reinterpret_cast<const float4*>(&s_b[k * 128 + 64 + tn * 4]);
            const float a[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
            const float b[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
#pragma unroll
            for (int i = 0; i < 8; ++i)
#pragma unroll
                for (int j = 0; j < 8; ++j) acc[i][j] = fmaf(b[j], a[i], acc[i][j]);
        }

        if (kQuantize) {
            __syncthreads();   // everyone has finished reading s_a: reuse it for the codes
            uint8_t* s_code = reinterpret_cast<uint8_t*>(s_a);   // [128 vectors][128 coords]
            const int nb = n_table;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                uint32_t lo = 0, hi = 0;
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    int c = 0;
                    for (int q = 0; q < nb; ++q) c += (acc[i][j] > s_table[q]) ? 1 : 0;
                    if (j < 4) lo |= (uint32_t)c << (8 * j);
                    else hi |= (uint32_t)c << (8 * (j - 4));
                }
                const int v = tm * 8 + i;
                *reinterpret_cast<uint32_t*>(&s_code[v * 128 + tn * 4]) = lo;
                *reinterpret_cast<uint32_t*>(&s_code[v * 128 + 64 + tn * 4]) = hi;
            }
            __syncthreads();
            const int total = kTileVecs * plen;
            for (int o = tid; o < total; o += kTileThreads) {
                const int v = o / plen, bi = o - v * plen;
                if (v0 + v < p.n_vec) {
                    uint32_t byte = 0;
                    for (int q = 0; q < vpb; ++q) byte |= (uint32_t)s_code[v * 128 + bi * vpb + q] << (q * bw);
                    p.indices[(v0 + v) * plen + bi] = (uint8_t)byte;
                }
            }
            if (tid < kTileVecs && v0 + tid < p.n_vec) p.norms[v0 + tid] = s_norm[tid];
        } else {
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const int v = tm * 8 + i;
                const long long gv = v0 + v;
                if (gv >= p.n_vec) continue;
                const float n = s_norm[v];
                float r[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) r[j] = acc[i][j] * n;
                if (p.out_dtype == 1) {
                    float* o = static_cast<float*>(p.out) + gv * kDim;
                    *reinterpret_cast<float4*>(o + tn * 4) = make_float4(r[0], r[1], r[2], r[3]);
                    *reinterpret_cast<float4*>(o + 64 + tn * 4) = make_float4(r[4], r[5], r[6], r[7]);
                } else {
                    __half* o = static_cast<__half*>(p.out) + gv * kDim;
                    __half2 h[4] = {__floats2half2_rn(r[0], r[1]), __floats2half2_rn(r[2], r[3]),
                                    __floats2half2_rn(r[4], r[5]), __floats2half2_rn(r[6], r[7])};
                    *reinterpret_cast<uint2*>(o + tn * 4) = *reinterpret_cast<uint2*>(&h[0]);
                    *reinterpret_cast<uint2*>(o + 64 + tn * 4) = *reinterpret_cast<uint2*>(&h[2]);
                }
            }
        }
    }
}

// ---------------------------------------------------------------------------
// Pool append: one CTA quantizes the new tokens that fall into one page of one
// (sequence, head, K|V) and writes them in the chunk layout of tq_layout.cuh.
// ---------------------------------------------------------------------------
struct AppendParams {
    const __half* k;
    const __half* v;
    int B, H, T_new;
    const float* Pi_k;
    const float* Pi_v;
    const float* bounds;
    uint8_t* pool;
    int n_pages;
    const int32_t* kv_indptr;
    const int32_t* kv_page_indices;
    const int32_t* start_pos;
};

template <int kTok>   // register accumulators per thread: 1 (single-token decode) or 16
__global__ void __launch_bounds__(128) tq_pool_append_kernel(const AppendParams p) {
    __shared__ __align__(16) float s_u[kDim][kTok];      // [k][token slot in this CTA]
    __shared__ uint8_t s_code[kTok][kDim];
    __shared__ float s_norm[kTok];
    __shared__ float s_bounds[8];

    pdl_begin();
    const int tid = threadIdx.x;
    const int b = blockIdx.x / p.H, h = blockIdx.x % p.H;
    const int which = blockIdx.z;                         // 0 = K, 1 = V
    const int pos0 = p.start_pos[b];
    const int page_ord = pos0 / 16 + blockIdx.y;          // page ordinal inside the sequence
    const int first = max(pos0, page_ord * 16);           // first / last+1 absolute positions handled here
    const int last = min(pos0 + p.T_new, page_ord * 16 + 16);
    const int nt = last - first;
    if (nt <= 0) return;
    const int slot0 = first - page_ord * 16;
    const int page = p.kv_page_indices[p.kv_indptr[b] + page_ord];
    if (page < 0 || page >= p.n_pages) return;            // invalid table entry: write nothing

    if (tid < 8) s_bounds[tid] = tid < 7 ? p.bounds[tid] : __int_as_float(0x7f800000);

    const __half* src = (which == 0 ? p.k : p.v) + (((size_t)b * p.H + h) * p.T_new + (first - pos0)) * kDim;
    const float* Pi = which == 0 ? p.Pi_k : p.Pi_v;

    // norms and unit vectors: two threads per token, 64 coordinates each
    if (tid < 2 * kTok) {
        const int t = tid >> 1, hf = tid & 1;
        float xr[64];
        if (t < nt) {
            const uint4* s4 = reinterpret_cast<const uint4*>(src + (size_t)t * kDim + hf * 64);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const uint4 w = __ldg(s4 + i);
                const float2 a = h2_to_f2(w.x), bb = h2_to_f2(w.y), c = h2_to_f2(w.z), d = h2_to_f2(w.w);
                xr[8 * i + 0] = a.x; xr[8 * i + 1] = a.y; xr[8 * i + 2] = bb.x; xr[8 * i + 3] = bb.y;
                xr[8 * i + 4] = c.x; xr[8 * i + 5] = c.y; xr[8 * i + 6] = d.x; xr[8 * i + 7] = d.y;
            }
        } else {
#pragma unroll
            for (int i = 0; i < 64; ++i) xr[i] = 0.f;
        }
        const double mine = sumsq64(xr);
        // only the 2 * kTok lanes inside this branch take part in the exchange
        constexpr unsigned kPairMask = kTok >= 16 ? 0xffffffffu : ((1u << (2 * kTok)) - 1u);
        const double other = __shfl_xor_sync(kPairMask, mine, 1);
        const double tot = hf == 0 ? mine + other : other + mine;
        const float norm = (float)sqrt(tot);
        const float denom = norm + 1e-10f;
        if (hf == 0) s_norm[t] = norm;
#pragma unroll
        for (int i = 0; i < 64; ++i) s_u[hf * 64 + i][t] = xr[i] / denom;
    }
    __syncthreads();

    // rotation: thread j owns output coordinate j for every token of the CTA
    {
        const int j = tid;
        float acc[kTok];
#pragma unroll
        for (int t = 0; t < kTok; ++t) acc[t] = 0.f;
        const float4* row = reinterpret_cast<const float4*>(Pi + (size_t)j * kDim);
#pragma unroll 2
        for (int k4 = 0; k4 < kDim / 4; ++k4) {
            const float4 pv = __ldg(row + k4);
            const float pk[4] = {pv.x, pv.y, pv.z, pv.w};
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const int k = 4 * k4 + q;
#pragma unroll
                for (int t = 0; t < kTok; ++t) acc[t] = fmaf(pk[q], s_u[k][t], acc[t]);
            }
        }
#pragma unroll
        for (int t = 0; t < kTok; ++t) {
            int c = 0;
#pragma unroll
            for (int q = 0; q < 7; ++q) c += (acc[t] > s_bounds[q]) ? 1 : 0;
            s_code[t][j] = (uint8_t)c;
        }
    }
    __syncthreads();

    uint8_t* chunk = p.pool + (((size_t)page * 2 + which) * p.H + h) * kChunkBytes;
    uint32_t* words = reinterpret_cast<uint32_t*>(chunk);
    __half* norms = reinterpret_cast<__half*>(chunk + kNormOffsetBytes);

    if (tid < nt) norms[slot0 + tid] = __float2half_rn(s_norm[tid]);

    for (int w = tid; w < kChunkWords; w += 128) {
        const int kk = w >> 6, ui = w & 63;
        if (which == 0) {
            const int slot = ui >> 2, t4 = ui & 3;
            const int t = slot - slot0;
            if (t < 0 || t >= nt) continue;
            uint32_t bits = 0;
#pragma unroll 8
            for (int e = 0; e < 32; ++e) bits |= unit_word_bits(e, kk, s_code[t][32 * t4 + e]);
            words[w] = bits;
        } else {
            const int pr = ui < 32 ? (ui & 3) : 4 + (ui & 3);
            const int g = (ui & 31) >> 2;
            const int ta = 2 * pr - slot0, tb = ta + 1;           // CTA-local token indices of the pair
            const bool has_a = ta >= 0 && ta < nt, has_b = tb >= 0 && tb < nt;
            if (!has_a && !has_b) continue;
            uint32_t bits = 0;
#pragma unroll 8
            for (int c = 0; c < 16; ++c) {
                if (has_a) bits |= unit_word_bits(2 * c, kk, s_code[ta][16 * g + c]);
                if (has_b) bits |= unit_word_bits(2 * c + 1, kk, s_code[tb][16 * g + c]);
            }
            if (!(has_a && has_b)) {
                // the other token of the pair was (or will be) written by another launch
                const uint32_t keep = has_a ? 0xF0F0F0F0u : 0x0F0F0F0Fu;
                bits |= words[w] & keep;
            }
            words[w] = bits;
        }
    }
}

#include "tq_append_tc.cuh"
#include "tq_append_t5.cuh"

// Coordinates decided by the exact chain / coordinates quantized by the tensor-core append, per device,
// since the last reset (read by leankv_tq_band_stats).
__device__ unsigned long long g_band_stats[2];
// Non-zero once a bounded wait for the tensor cores inside the tcgen05 append has run out (per device, sticky;
// read by leankv_tq_append_status).
__device__ int g_append_status;

struct UnpackParams {
    const uint8_t* pool;
    int n_pages, H;
    const int32_t* page_indices;
    int n_tokens, which;
    uint8_t* indices;
    float* norms;
};

__global__ void tq_pool_unpack_kernel(const UnpackParams p) {
    const long long total = (long long)p.H * p.n_tokens * 64;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        const int byte = (int)(i & 63);
        const long long ht = i >> 6;
        const int tok = (int)(ht % p.n_tokens), h = (int)(ht / p.n_tokens);
        const int page = p.page_indices[tok >> 4], slot = tok & 15;
        if (page < 0 || page >= p.n_pages) {
            // a stale or foreign page id: nothing is read from the pool; the token reads as code 0, norm 0
            p.indices[i] = 0;
            if (byte == 0) p.norms[ht] = 0.f;
            continue;
        }
        const uint8_t* chunk = p.pool + (((size_t)page * 2 + p.which) * p.H + h) * kChunkBytes;
        const uint32_t* words = reinterpret_cast<const uint32_t*>(chunk);
        const int c0 = 2 * byte, c1 = c0 + 1;
        const int lo = chunk_get_code(words, p.which == 0 ? k_code_slot(slot, c0) : v_code_slot(slot, c0));
        const int hi = chunk_get_code(words, p.which == 0 ? k_code_slot(slot, c1) : v_code_slot(slot, c1));
        p.indices[i] = (uint8_t)(lo | (hi << 4));
        if (byte == 0)
            p.norms[ht] = __half2float(reinterpret_cast<const __half*>(chunk + kNormOffsetBytes)[slot]);
    }
}

// LEANKV_TQ_APPEND selects the kernel of multi-token appends: "fp32" = the fp32 kernel (the definition the
// tensor-core paths are tested against), default / "mma" = fast rotation on mma.sync (64-token tiles, two CTAs
// per SM), "t5" = fast rotation on tcgen05 (128-token tiles, one CTA per SM: measured slower, 1.49 ms against
// 1.09 ms for a million vectors, because its norm / code / pack phases have no second CTA to overlap with).
// All three write the same bits.
int tc_append_mode() {
    static int state = -1;
    if (state < 0) {
        const char* e = std::getenv("LEANKV_TQ_APPEND");
        state = e == nullptr ? 1 : (e[0] == 'f' ? 0 : (e[0] == 't' && e[1] == '5' ? 2 : 1));
    }
    return state;
}
bool tc_append_enabled() { return tc_append_mode() != 0; }

int check_tq_common(long long n_vec, int dim, int bits) {
    if (n_vec < 0) return LEANKV_EINVAL;
    if (dim != kDim) return LEANKV_EUNSUPPORTED;
    if (bits < 1 || bits > 4) return LEANKV_EUNSUPPORTED;
    return LEANKV_OK;
}

template <bool kQuantize>
int launch_tile(const TileParams& p, void* stream) {
    // The opt-in to 128 KiB of dynamic shared memory belongs to a device's copy of the function, so it is
    // remembered per device ordinal (a process may quantize on several GPUs). Racing first calls all
    // store the same value.
    constexpr int kMaxDevices = 64;
    static bool attr_done[kMaxDevices][2] = {};
    int dev = 0;
    LEANKV_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= kMaxDevices || !attr_done[dev][kQuantize]) {
        LEANKV_CUDA_TRY(cudaFuncSetAttribute(tq_tile_kernel<kQuantize>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             (int)kTileSmemBytes));
        if (dev >= 0 && dev < kMaxDevices) attr_done[dev][kQuantize] = true;
    }
    const long long n_tiles = (p.n_vec + kTileVecs - 1) / kTileVecs;
    const int grid = (int)(n_tiles < sm_count() ? n_tiles : sm_count());
    tq_tile_kernel<kQuantize><<<grid, kTileThreads, kTileSmemBytes, static_cast<cudaStream_t>(stream)>>>(p);
    LEANKV_CUDA_TRY(cudaGetLastError());
    return LEANKV_OK;
}

}  // namespace
}  // namespace leankv

using namespace leankv;

extern "C" int leankv_tq_packed_len(int dim, int bits) {
    if (dim <= 0 || bits < 1) return LEANKV_EINVAL;
    const int vpb = bits == 1 ? 8 : bits == 2 ? 4 : bits <= 4 ? 2 : 1;
    return (dim + vpb - 1) / vpb;
}

extern "C" int leankv_tq_quantize(const void* x, int x_dtype, long long n_vec, int dim, int bits,
                                  const float* Pi, const float* decision_boundaries,
                                  uint8_t* indices, float* norms, void* stream) {
    int rc = check_tq_common(n_vec, dim, bits);
    if (rc != LEANKV_OK) return rc;
    if (n_vec == 0) return LEANKV_OK;
    if (!x || !Pi || !decision_boundaries || !indices || !norms) return LEANKV_EINVAL;
    if (x_dtype != 0 && x_dtype != 1) return LEANKV_EINVAL;
    if (!aligned16(x) || !aligned16(Pi)) return LEANKV_EALIGN;
    TileParams p{};
    p.x = x;
    p.x_dtype = x_dtype;
    p.n_vec = n_vec;
    p.bits = bits;
    p.Pi = Pi;
    p.table = decision_boundaries;
    p.indices = indices;
    p.norms = norms;
    return launch_tile<true>(p, stream);
}

extern "C" int leankv_tq_dequantize(const uint8_t* indices, const float* norms, long long n_vec,
                                    int dim, int bits, const float* Pi, const float* centroids,
                                    void* x_hat, int out_dtype, void* stream) {
    int rc = check_tq_common(n_vec, dim, bits);
    if (rc != LEANKV_OK) return rc;
    if (n_vec == 0) return LEANKV_OK;
    if (!indices || !norms || !Pi || !centroids || !x_hat) return LEANKV_EINVAL;
    if (out_dtype != 0 && out_dtype != 1) return LEANKV_EINVAL;
    if (!aligned16(x_hat) || !aligned16(Pi)) return LEANKV_EALIGN;
    TileParams p{};
    p.n_vec = n_vec;
    p.bits = bits;
    p.Pi = Pi;
    p.table = centroids;
    p.indices = const_cast<uint8_t*>(indices);
    p.norms = const_cast<float*>(norms);
    p.out = x_hat;
    p.out_dtype = out_dtype;
    return launch_tile<false>(p, stream);
}

extern "C" size_t leankv_tq_pool_bytes(int n_pages, int n_kv_heads) {
    if (n_pages <= 0 || n_kv_heads <= 0) return 0;
    return (size_t)n_pages * 2 * n_kv_heads * kChunkBytes;
}

extern "C" int leankv_tq_pool_append(const void* k, const void* v, int B, int n_kv_heads, int T_new,
                                     const float* Pi_k, const float* Pi_v,
                                     const float* decision_boundaries, void* pool, int n_pages,
                                     const int32_t* kv_indptr, const int32_t* kv_page_indices,
                                     const int32_t* start_pos, void* stream) {
    if (B < 0 || n_kv_heads <= 0 || T_new < 0 || n_pages <= 0) return LEANKV_EINVAL;
    if (B == 0 || T_new == 0) return LEANKV_OK;
    if (!k || !v || !Pi_k || !Pi_v || !decision_boundaries || !pool || !kv_indptr ||
        !kv_page_indices || !start_pos)
        return LEANKV_EINVAL;
    if (!aligned16(k) || !aligned16(v) || !aligned16(Pi_k) || !aligned16(Pi_v) || !aligned16(pool))
        return LEANKV_EALIGN;
    if ((long long)B * n_kv_heads > 0x7fffffffLL) return LEANKV_ELIMIT;
    AppendParams p{};
    p.k = static_cast<const __half*>(k);
    p.v = static_cast<const __half*>(v);
    p.B = B;
    p.H = n_kv_heads;
    p.T_new = T_new;
    p.Pi_k = Pi_k;
    p.Pi_v = Pi_v;
    p.bounds = decision_boundaries;
    p.pool = static_cast<uint8_t*>(pool);
    p.n_pages = n_pages;
    p.kv_indptr = kv_indptr;
    p.kv_page_indices = kv_page_indices;
    p.start_pos = start_pos;
    // T_new tokens starting anywhere inside a page touch at most (T_new + 14) / 16 + 1 pages.
    const int groups = (T_new + 14) / 16 + 1;
    if (T_new >= 16 && tc_append_enabled()) {
        // prompt-sized appends: rotation on tensor cores, codes identical to the fp32 kernels
        AppendTcParams tp{};
        tp.a = p;
        const bool t5 = tc_append_mode() == 2;
        const int pages_per_tile = t5 ? kT5Pages : 4;
        tp.groups = (groups + pages_per_tile - 1) / pages_per_tile;
        tp.n_tiles = 2LL * B * n_kv_heads * tp.groups;
        void* stats = nullptr;
        LEANKV_CUDA_TRY(cudaGetSymbolAddress(&stats, g_band_stats));
        tp.stats = static_cast<unsigned long long*>(stats);
        int dev = 0;
        LEANKV_CUDA_TRY(cudaGetDevice(&dev));
        constexpr int kMaxDevices = 64;
        static bool attr_done[kMaxDevices] = {};
        if (dev < 0 || dev >= kMaxDevices || !attr_done[dev]) {
            LEANKV_CUDA_TRY(cudaFuncSetAttribute(tq_pool_append_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                 (int)kTcSmemBytes));
            LEANKV_CUDA_TRY(cudaFuncSetAttribute(tq_pool_append_t5_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                 (int)kT5SmemBytes));
            if (dev >= 0 && dev < kMaxDevices) attr_done[dev] = true;
        }
        if (t5) {
            void* st_word = nullptr;
            LEANKV_CUDA_TRY(cudaGetSymbolAddress(&st_word, g_append_status));
            const long long slots1 = sm_count();            // 148 KB of shared memory: one CTA per SM
            const int grid_t5 = (int)(tp.n_tiles < slots1 ? tp.n_tiles : slots1);
            LEANKV_CUDA_TRY(launch_kernel(tq_pool_append_t5_kernel, dim3(grid_t5), dim3(kT5Threads), kT5SmemBytes,
                                          static_cast<cudaStream_t>(stream), tp, static_cast<int*>(st_word)));
            return LEANKV_OK;
        }
        const long long slots = 2LL * sm_count();
        const int grid_tc = (int)(tp.n_tiles < slots ? tp.n_tiles : slots);
        LEANKV_CUDA_TRY(launch_kernel(tq_pool_append_tc_kernel, dim3(grid_tc), dim3(kTcThreads), kTcSmemBytes,
                                      static_cast<cudaStream_t>(stream), tp));
        return LEANKV_OK;
    }
    if (groups > 65535) return LEANKV_ELIMIT;
    dim3 grid(B * n_kv_heads, groups, 2);
    if (T_new == 1)
        LEANKV_CUDA_TRY(launch_kernel(tq_pool_append_kernel<1>, grid, dim3(128), 0, static_cast<cudaStream_t>(stream), p));
    else
        LEANKV_CUDA_TRY(launch_kernel(tq_pool_append_kernel<16>, grid, dim3(128), 0, static_cast<cudaStream_t>(stream), p));
    return LEANKV_OK;
}

extern "C" int leankv_tq_pool_unpack(const void* pool, int n_pages, int n_kv_heads,
                                     const int32_t* page_indices, int n_tokens, int which,
                                     uint8_t* indices, float* norms, void* stream) {
    if (n_pages <= 0 || n_kv_heads <= 0 || n_tokens < 0 || (which != 0 && which != 1))
        return LEANKV_EINVAL;
    if (n_tokens == 0) return LEANKV_OK;
    if (!pool || !page_indices || !indices || !norms) return LEANKV_EINVAL;
    UnpackParams p{};
    p.pool = static_cast<const uint8_t*>(pool);
    p.n_pages = n_pages;
    p.H = n_kv_heads;
    p.page_indices = page_indices;
    p.n_tokens = n_tokens;
    p.which = which;
    p.indices = indices;
    p.norms = norms;
    const long long total = (long long)n_kv_heads * n_tokens * 64;
    long long blocks = (total + 255) / 256;
    if (blocks > sm_count() * 16LL) blocks = sm_count() * 16LL;
    tq_pool_unpack_kernel<<<(int)blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(p);
    LEANKV_CUDA_TRY(cudaGetLastError());
    return LEANKV_OK;
}

extern "C" int leankv_tq_append_status(int* status /* host */) {
    if (!status) return LEANKV_EINVAL;
    LEANKV_CUDA_TRY(cudaMemcpyFromSymbol(status, g_append_status, sizeof(int)));
    return LEANKV_OK;
}

extern "C" int leankv_tq_band_stats(unsigned long long* stats /* host, 2 */, int reset) {
    if (!stats) return LEANKV_EINVAL;
    LEANKV_CUDA_TRY(cudaMemcpyFromSymbol(stats, g_band_stats, sizeof(unsigned long long) * 2));
    if (reset) {
        const unsigned long long zero[2] = {0ull, 0ull};
        LEANKV_CUDA_TRY(cudaMemcpyToSymbol(g_band_stats, zero, sizeof(zero)));
    }
    return LEANKV_OK;
}
