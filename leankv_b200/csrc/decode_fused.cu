// One launch for everything between the fused q/k/v projection and attention in a decode step
// (one new token per sequence): rotary embedding of q and k, rotation of q into the key codebook's space, and
// rotate + Lloyd-Max quantize + 3-bit pack of the new k and v into their page.
//
// It produces bit for bit what leankv_rope_f16 + leankv_tq_pool_append (T_new = 1) +
// the query rotation of leankv_tq_decode_attn produce as three launches: same fp16 rounding
// points for the rotary step, same norm / division / ascending-k fma order for the rotations
// (the arithmetic contract stated at the top of tq_quantize.cu).

#include <algorithm>

#include "common.cuh"
#include "tq_layout.cuh"

namespace leankv {
namespace {

constexpr int kDim = LEANKV_TQ_DIM;

struct PostParams {
    const __half* qkv;        // [B][(nq + 2 nkv) * 128]
    const float* inv_freq;
    const int* pos;           // [B] position of the token being decoded
    const int* kv_indptr;     // [B + 1] offsets into page_indices, or nullptr (one sequence at offset 0)
    int B;
    const float* Pi_k_t;   // transposes of the rotations: Pi_k_t[k][j] = Pi_k[j][k]
    const float* Pi_v_t;
    const float* bounds;
    uint8_t* pool;
    int n_pages;
    const int32_t* page_indices;
    int nq, nkv;
    float* q_rot;             // [B][nq][128]
};

__global__ void __launch_bounds__(kDim) decode_qkv_post_kernel(const PostParams p) {
    __shared__ float s_x[kDim];       // the head vector (after rotary embedding, fp16 values)
    __shared__ float s_u[kDim];       // what gets rotated: x for q, x / (norm + 1e-10) for k and v
    __shared__ double s_ss[2];
    __shared__ float s_bounds[8];
    __shared__ __align__(4) uint8_t s_code[kDim];

    const int j = threadIdx.x;
    const int head = blockIdx.x;
    const int kind = head < p.nq ? 0 : (head < p.nq + p.nkv ? 1 : 2);   // 0 q, 1 k, 2 v
    // The rotation matrix is a constant of the cache, not an output of the previous kernel: fetch this
    // thread's column of it right away (128 independent loads, one memory round trip) so that it
    // is in registers by the time the vector has been prepared.
    const float* PiT = kind == 2 ? p.Pi_v_t : p.Pi_k_t;
    float pi_col[kDim];
#pragma unroll
    for (int k = 0; k < kDim; ++k) pi_col[k] = __ldg(PiT + k * kDim + j);
    pdl_begin();
    if (j < 8) s_bounds[j] = j < 7 ? p.bounds[j] : __int_as_float(0x7f800000);
    const int row = (p.nq + 2 * p.nkv) * kDim;

    // One CTA serves its head for every gridDim.y-th sequence with the rotation column held in registers.
    for (int b = blockIdx.y; b < p.B; b += gridDim.y) {
        const int pos = p.pos[b];
        const __half* src = p.qkv + (size_t)b * row + (size_t)head * kDim;
        // where the new token goes: fetched now so that the page-table round trip (and, for V, the word
        // shared with the pair token) overlaps the arithmetic instead of trailing it
        const int which = kind - 1;
        const int h = which == 0 ? head - p.nq : head - p.nq - p.nkv;
        const int slot = pos & 15;
        int page = -1;
        uint32_t* words = nullptr;
        uint32_t old_word = 0;
        if (kind != 0) {
            const int base = p.kv_indptr != nullptr ? p.kv_indptr[b] : 0;
            page = p.page_indices[base + (pos >> 4)];
            if (page >= 0 && page < p.n_pages) {
                words = reinterpret_cast<uint32_t*>(p.pool + (((size_t)page * 2 + which) * p.nkv + h) * kChunkBytes);
                if (which == 1 && j < 24) {
                    const int g = j & 7, kk = j >> 3, pr = slot >> 1;
                    old_word = words[kk * 64 + (pr < 4 ? 4 * g + pr : 32 + 4 * g + (pr - 4))];
                }
            }
        }

        __half xv = src[j];
        if (kind != 2) {
            // rotate_half form: out[i] = x[i] cos - x[i+64] sin ; out[i+64] = x[i+64] cos + x[i] sin,
            // cos/sin rounded to fp16, products and sum in fp16 (HF apply_rotary_pos_emb)
            const int i = j & 63;
            const float ang = (float)pos * p.inv_freq[i];
            const __half c = __float2half_rn(cosf(ang)), s = __float2half_rn(sinf(ang));
            const __half other = src[j ^ 64];
            xv = j < 64 ? __hadd(__hmul(xv, c), __hmul(__hneg(other), s))
                        : __hadd(__hmul(xv, c), __hmul(other, s));
        }
        const float xf = __half2float(xv);
        __syncthreads();                       // the previous sequence's readers of s_x / s_u / s_code are done
        s_x[j] = xf;
        __syncthreads();

        float norm = 0.f;
        if (kind != 0) {
            // fp64 sums of squares of coordinates 0..63 and 64..127, ascending (one thread each)
            if ((j & 63) == 0) {
                double ss = 0.0;
#pragma unroll 8
                for (int k = 0; k < 64; ++k) {
                    const double v = (double)s_x[j + k];
                    ss = fma(v, v, ss);
                }
                s_ss[j >> 6] = ss;
            }
            __syncthreads();
            norm = (float)sqrt(s_ss[0] + s_ss[1]);
            s_u[j] = xf / (norm + 1e-10f);
        } else {
            s_u[j] = xf;
        }
        __syncthreads();

        // y_j = sum_k Pi[j][k] u[k], k ascending
        float y = 0.f;
#pragma unroll
        for (int k = 0; k < kDim; ++k) y = fmaf(pi_col[k], s_u[k], y);
        if (kind == 0) {
            p.q_rot[((size_t)b * p.nq + head) * kDim + j] = y;
            continue;
        }
        int code = 0;
#pragma unroll
        for (int q = 0; q < 7; ++q) code += (y > s_bounds[q]) ? 1 : 0;
        s_code[j] = (uint8_t)code;
        __syncthreads();

        if (words == nullptr) continue;
        uint8_t* chunk = reinterpret_cast<uint8_t*>(words);
        if (j == 0) reinterpret_cast<__half*>(chunk + kNormOffsetBytes)[slot] = __float2half_rn(norm);

        // four codes per 32-bit shared-memory load; pack4 squeezes the low nibbles of 4 bytes into 16 bits
        auto pack4 = [](uint32_t v) -> uint32_t {
            const uint32_t t2 = (v | (v >> 4)) & 0x00FF00FFu;
            return (t2 | (t2 >> 8)) & 0xFFFFu;
        };
        if (which == 0) {
            if (j < 12) {                      // 4 units (quarters of the vector) x 3 words, this token only
                const int t4 = j & 3, kk = j >> 2;
                const uint32_t* c4 = reinterpret_cast<const uint32_t*>(&s_code[32 * t4]);
                const uint32_t lo = c4[2 * kk] & 0x07070707u, hi = c4[2 * kk + 1] & 0x07070707u;
                const uint32_t s_lo = ((c4[6] >> kk) & 0x01010101u) << 3, s_hi = ((c4[7] >> kk) & 0x01010101u) << 3;
                words[kk * 64 + slot * 4 + t4] = pack4(lo) | (pack4(hi) << 16) | pack4(s_lo) | (pack4(s_hi) << 16);
            }
        } else {
            if (j < 24) {                      // 8 units (16-coordinate groups) x 3 words, shared with the pair token
                const int g = j & 7, kk = j >> 3;
                const int pr = slot >> 1, par = slot & 1;
                const int ui = pr < 4 ? 4 * g + pr : 32 + 4 * g + (pr - 4);
                const uint32_t* ca = reinterpret_cast<const uint32_t*>(&s_code[16 * g]);
                const uint32_t a4 = ca[kk] & 0x07070707u, as4 = (ca[3] >> kk) & 0x01010101u;
                const uint32_t bits = par ? ((a4 << 4) | (as4 << 7)) : (a4 | (as4 << 3));
                const uint32_t keep = par ? 0x0F0F0F0Fu : 0xF0F0F0F0u;   // the other token's nibbles
                words[kk * 64 + ui] = bits | (old_word & keep);
            }
        }
    }
}

}  // namespace
}  // namespace leankv

using namespace leankv;

static int post_launch(const void* qkv, int B, const float* inv_freq, const int32_t* pos,
                       const int32_t* kv_indptr, const float* Pi_k_t, const float* Pi_v_t,
                       const float* decision_boundaries, void* pool, int n_pages, const int32_t* page_indices,
                       int n_q_heads, int n_kv_heads, float* q_rot, void* stream) {
    if (!qkv || !inv_freq || !pos || !Pi_k_t || !Pi_v_t || !decision_boundaries || !pool || !page_indices ||
        !q_rot || n_pages <= 0 || n_q_heads <= 0 || n_kv_heads <= 0 || B <= 0)
        return LEANKV_EINVAL;
    if (!aligned16(pool)) return LEANKV_EALIGN;
    PostParams p{};
    p.qkv = static_cast<const __half*>(qkv);
    p.inv_freq = inv_freq;
    p.pos = pos;
    p.kv_indptr = kv_indptr;
    p.B = B;
    p.Pi_k_t = Pi_k_t;
    p.Pi_v_t = Pi_v_t;
    p.bounds = decision_boundaries;
    p.pool = static_cast<uint8_t*>(pool);
    p.n_pages = n_pages;
    p.page_indices = page_indices;
    p.nq = n_q_heads;
    p.nkv = n_kv_heads;
    p.q_rot = q_rot;
    // enough CTAs to fill the GPU a few times over, each reusing its rotation column for ~8 sequences
    const int heads = n_q_heads + 2 * n_kv_heads;
    const int gy = std::max(1, std::min(B, (B + 7) / 8));
    LEANKV_CUDA_TRY(launch_kernel_ex(true, decode_qkv_post_kernel, dim3(heads, gy), dim3(kDim), 0,
                                     static_cast<cudaStream_t>(stream), p));
    return LEANKV_OK;
}

extern "C" int leankv_decode_qkv_post(const void* qkv, const float* inv_freq, const int32_t* state,
                                      const float* Pi_k_t, const float* Pi_v_t,
                                      const float* decision_boundaries, void* pool, int n_pages,
                                      const int32_t* page_indices, int n_q_heads, int n_kv_heads,
                                      float* q_rot, void* stream) {
    return post_launch(qkv, 1, inv_freq, state /* state[0] = position */, nullptr, Pi_k_t, Pi_v_t,
                       decision_boundaries, pool, n_pages, page_indices, n_q_heads, n_kv_heads, q_rot, stream);
}

extern "C" int leankv_batch_qkv_post(const void* qkv, int B, const float* inv_freq, const int32_t* pos,
                                     const int32_t* kv_indptr, const float* Pi_k_t, const float* Pi_v_t,
                                     const float* decision_boundaries, void* pool, int n_pages,
                                     const int32_t* kv_page_indices, int n_q_heads, int n_kv_heads,
                                     float* q_rot, void* stream) {
    if (!kv_indptr) return LEANKV_EINVAL;
    return post_launch(qkv, B, inv_freq, pos, kv_indptr, Pi_k_t, Pi_v_t, decision_boundaries, pool, n_pages,
                       kv_page_indices, n_q_heads, n_kv_heads, q_rot, stream);
}
