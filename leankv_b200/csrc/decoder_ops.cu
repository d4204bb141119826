// Small kernels that sit between the two hot paths in a batch-1 decode step of a
// Llama/Mistral-style block: embedding fetch, RMSNorm, rotary embedding, greedy argmax and
// the on-device bookkeeping of the sequence position / page table, so that a whole decode
// step can be replayed as one CUDA graph without the host touching per-step values.
// Rounding points follow the HF eager modules the reference runs around its kernels
// (transformers modeling_mistral.py: MistralRMSNorm, apply_rotary_pos_emb).

#include <algorithm>

#include "common.cuh"

namespace leankv {
namespace {

// Decode state words (int32[8], device), as the header describes them beside leankv_decode_begin: position,
// step count, and the one-sequence page table (kv_indptr[0..1], kv_last_page_len, start position).
enum { kPos = 0, kStep = 1, kIndptr0 = 2, kIndptr1 = 3, kLastLen = 4, kStartPos = 5 };

__device__ __forceinline__ float block_sum(float v, float* s_tmp) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    if (lane == 0) s_tmp[warp] = v;
    __syncthreads();
    const int nw = (blockDim.x + 31) >> 5;
    float t = 0.f;
    for (int w = 0; w < nw; ++w) t += s_tmp[w];   // fixed order: bit-reproducible
    __syncthreads();
    return t;
}

// Optional residual update h += delta (fp16 add, as the decoder block does), then
// y = w * fp16( h * rsqrt(mean(h^2) + eps) ), statistics in fp32.
// One CTA per row; 16-byte accesses; the (updated) row stays in registers between the two phases
// (n % 8 == 0, n <= kNormThreads * 8 * kNormVecs).
constexpr int kNormThreads = 512;
constexpr int kNormVecs = 4;
__global__ void __launch_bounds__(kNormThreads) rmsnorm_kernel(__half* x, const __half* delta,
                                                               const __half* w, __half* y, int n, float eps) {
    __shared__ float s_tmp[32];
    pdl_begin();
    const int nvec = n >> 3;
    x += (size_t)blockIdx.x * n;
    y += (size_t)blockIdx.x * n;
    if (delta != nullptr) delta += (size_t)blockIdx.x * n;
    uint4 v[kNormVecs];
    float ss = 0.f;
#pragma unroll
    for (int it = 0; it < kNormVecs; ++it) {
        const int i = threadIdx.x + it * kNormThreads;
        if (i < nvec) {
            uint4 a = reinterpret_cast<const uint4*>(x)[i];
            if (delta != nullptr) {
                const uint4 d = __ldg(reinterpret_cast<const uint4*>(delta) + i);
                __half2* ah = reinterpret_cast<__half2*>(&a);
                const __half2* dh = reinterpret_cast<const __half2*>(&d);
#pragma unroll
                for (int q = 0; q < 4; ++q) ah[q] = __hadd2(ah[q], dh[q]);
                reinterpret_cast<uint4*>(x)[i] = a;
            }
            v[it] = a;
            const __half2* ah = reinterpret_cast<const __half2*>(&a);
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const float2 f = __half22float2(ah[q]);
                ss = fmaf(f.x, f.x, ss);
                ss = fmaf(f.y, f.y, ss);
            }
        }
    }
    const float tot = block_sum(ss, s_tmp);
    const float r = rsqrtf(tot / (float)n + eps);
#pragma unroll
    for (int it = 0; it < kNormVecs; ++it) {
        const int i = threadIdx.x + it * kNormThreads;
        if (i < nvec) {
            const uint4 wv = __ldg(reinterpret_cast<const uint4*>(w) + i);
            const __half2* ah = reinterpret_cast<const __half2*>(&v[it]);
            const __half2* wh = reinterpret_cast<const __half2*>(&wv);
            uint4 o;
            __half2* oh = reinterpret_cast<__half2*>(&o);
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const float2 f = __half22float2(ah[q]);
                oh[q] = __hmul2(wh[q], __floats2half2_rn(f.x * r, f.y * r));
            }
            reinterpret_cast<uint4*>(y)[i] = o;
        }
    }
}

// Fetch the embedding row of the current token and derive this step's page-table words.
__global__ void __launch_bounds__(256) decode_begin_kernel(const __half* table, const long long* token,
                                                           __half* h, int hidden, int vocab,
                                                           int* state) {
    pdl_begin();
    long long tok = *token;
    if (tok < 0 || tok >= vocab) tok = 0;
    const uint4* src = reinterpret_cast<const uint4*>(table + (size_t)tok * hidden);
    uint4* dst = reinterpret_cast<uint4*>(h);
    for (int i = threadIdx.x; i < hidden / 8; i += blockDim.x) dst[i] = __ldg(src + i);
    if (threadIdx.x == 0) {
        const int pos = state[kPos];
        state[kStartPos] = pos;
        state[kIndptr0] = 0;
        state[kIndptr1] = pos / 16 + 1;
        state[kLastLen] = pos % 16 + 1;
    }
}

// Rotary embedding (rotate_half form) on the q and k parts of a fused qkv row.
// cos/sin are rounded to fp16 and the products/sum are fp16, as in the HF module.
__global__ void __launch_bounds__(64) rope_kernel(const __half* qkv, const float* inv_freq,
                                                  const int* state, __half* q_out, __half* k_out,
                                                  int n_q_heads, int n_kv_heads) {
    pdl_begin();
    const int head = blockIdx.x;                 // q heads first, then k heads
    const int i = threadIdx.x;                   // 0..63
    const float ang = (float)state[kPos] * inv_freq[i];
    const __half c = __float2half_rn(cosf(ang)), s = __float2half_rn(sinf(ang));
    const __half* src = qkv + (size_t)head * 128;
    __half* dst = head < n_q_heads ? q_out + (size_t)head * 128
                                   : k_out + (size_t)(head - n_q_heads) * 128;
    const __half a = src[i], b = src[i + 64];
    dst[i] = __hadd(__hmul(a, c), __hmul(__hneg(b), s));
    dst[i + 64] = __hadd(__hmul(b, c), __hmul(a, s));
}

// Greedy next token (lowest index wins ties), appended to the history; advances the position.
// One CTA per sequence: pos / step are that sequence's words.
__global__ void __launch_bounds__(1024) decode_end_kernel(const __half* logits, int vocab,
                                                          long long* token, long long* history,
                                                          int history_cap, int* pos, int* step_ptr) {
    __shared__ float s_v[32];
    __shared__ int s_i[32];
    pdl_begin();
    logits += (size_t)blockIdx.x * vocab;
    token += blockIdx.x;
    history += (size_t)blockIdx.x * history_cap;
    pos += blockIdx.x;
    step_ptr += blockIdx.x;
    float best = -INFINITY;
    int best_i = 0x7fffffff;
    const int nvec = vocab >> 3;     // 16-byte loads; indices ascend within a thread, so '>' keeps the lowest
    for (int vi = threadIdx.x; vi < nvec; vi += blockDim.x) {
        const uint4 a = __ldg(reinterpret_cast<const uint4*>(logits) + vi);
        const __half* hp = reinterpret_cast<const __half*>(&a);
#pragma unroll
        for (int q = 0; q < 8; ++q) {
            const float v = __half2float(hp[q]);
            if (v > best) { best = v; best_i = vi * 8 + q; }
        }
    }
    for (int i = nvec * 8 + threadIdx.x; i < vocab; i += blockDim.x) {
        const float v = __half2float(logits[i]);
        if (v > best || (v == best && i < best_i)) { best = v; best_i = i; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
        if (ov > best || (ov == best && oi < best_i)) { best = ov; best_i = oi; }
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) { s_v[warp] = best; s_i[warp] = best_i; }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < (int)(blockDim.x >> 5); ++w)
            if (s_v[w] > best || (s_v[w] == best && s_i[w] < best_i)) { best = s_v[w]; best_i = s_i[w]; }
        if (best_i == 0x7fffffff) best_i = 0;   // all-NaN row
        *token = best_i;
        const int step = *step_ptr;
        if (step < history_cap) history[step] = best_i;
        *step_ptr = step + 1;
        *pos = *pos + 1;
    }
}

// The same for an output head that is split over the vocabulary among tensor-parallel ranks: every
// rank finds the best of its own slice, sends {value, index} (two 64-bit words, each tagged with the
// step's epoch like the partial sums of the row-parallel GEMV) to every rank's receive area, waits
// (bounded) for all ranks' words, and takes the largest value, lowest index on ties: every rank
// arrives at the same token. As the last exchange of a step it also moves the epoch on.
struct ShardedEndParams {
    const __half* logits;      // this rank's slice [vocab_local]
    int vocab_local, vocab_offset;
    long long* token;
    long long* history;
    int history_cap;
    int* pos;
    int* step_ptr;
    int world, rank, limit;
    unsigned long long* recv[LEANKV_MAX_RANKS];   // slot base in every rank's area: [world][2] words
    int* epoch;
    int* status;
};

__global__ void __launch_bounds__(1024) decode_end_sharded_kernel(const ShardedEndParams p) {
    __shared__ float s_v[32];
    __shared__ int s_i[32];
    pdl_begin();
    float best = -INFINITY;
    int best_i = 0x7fffffff;
    const int nvec = p.vocab_local >> 3;      // vocab_local % 8 == 0 (checked on the host)
    for (int vi = threadIdx.x; vi < nvec; vi += blockDim.x) {
        const uint4 a = __ldg(reinterpret_cast<const uint4*>(p.logits) + vi);
        const __half* hp = reinterpret_cast<const __half*>(&a);
#pragma unroll
        for (int q = 0; q < 8; ++q) {
            const float v = __half2float(hp[q]);
            if (v > best) { best = v; best_i = vi * 8 + q; }
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
        if (ov > best || (ov == best && oi < best_i)) { best = ov; best_i = oi; }
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) { s_v[warp] = best; s_i[warp] = best_i; }
    __syncthreads();
    if (threadIdx.x != 0) return;
    for (int w = 1; w < (int)(blockDim.x >> 5); ++w)
        if (s_v[w] > best || (s_v[w] == best && s_i[w] < best_i)) { best = s_v[w]; best_i = s_i[w]; }
    if (best_i != 0x7fffffff) best_i += p.vocab_offset;

    const unsigned int ep = (unsigned int)*reinterpret_cast<volatile int*>(p.epoch);
    const unsigned long long tag = (unsigned long long)ep << 32;
    for (int i = 0; i < p.world; ++i) {
        int r = p.rank + i;
        r = r >= p.world ? r - p.world : r;
        unsigned long long* dst = p.recv[r] + 2 * p.rank;
        asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(dst), "l"(tag | __float_as_uint(best)) : "memory");
        asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(dst + 1), "l"(tag | (unsigned int)best_i) : "memory");
    }
    const bool live = *reinterpret_cast<volatile int*>(p.status) == 0;
    bool ok = live;
    float top = -INFINITY;
    int top_i = 0x7fffffff;
    const unsigned long long* src = p.recv[p.rank];
    for (int r = 0; r < p.world && live; ++r) {
        unsigned long long wv = 0, wi = 0;
        int it = 0;
        for (;;) {
            asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(wv) : "l"(src + 2 * r) : "memory");
            asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(wi) : "l"(src + 2 * r + 1) : "memory");
            if (((unsigned int)(wv >> 32) == ep && (unsigned int)(wi >> 32) == ep) || it >= p.limit) break;
            __nanosleep(20);
            ++it;
        }
        if ((unsigned int)(wv >> 32) != ep || (unsigned int)(wi >> 32) != ep) {
            ok = false;
            continue;
        }
        const float v = __uint_as_float((unsigned int)wv);
        const int idx = (int)(unsigned int)wi;
        if (v > top || (v == top && idx < top_i)) { top = v; top_i = idx; }
    }
    if (!ok && live) atomicOr(p.status, 1);
    if (top_i == 0x7fffffff) top_i = 0;      // all-NaN rows, or a dead exchange
    *p.token = top_i;
    const int step = *p.step_ptr;
    if (step < p.history_cap) p.history[step] = top_i;
    *p.step_ptr = step + 1;
    *p.pos = *p.pos + 1;
    *p.epoch = (int)(ep + 1u);
}

// Batched step prologue: embedding rows of B tokens, and the flat page table of this step built from
// a per-sequence block table. Sequence b caches pos[b] tokens and appends one: it uses
// pos[b] / 16 + 1 pages, the first entries of block_table[b][0..max_pps). One CTA per sequence; each
// derives its own offset from the positions of the sequences before it, so no CTA waits on another.
__global__ void __launch_bounds__(256) batch_begin_kernel(const __half* table, const long long* tokens,
                                                          __half* h, int hidden, int vocab, int B,
                                                          const int* pos, const int* block_table, int max_pps,
                                                          int* kv_indptr, int* kv_page_indices,
                                                          int* kv_last_page_len) {
    __shared__ int s_part[8];
    pdl_begin();
    const int b = blockIdx.x;
    long long tok = tokens[b];
    if (tok < 0 || tok >= vocab) tok = 0;
    const uint4* src = reinterpret_cast<const uint4*>(table + (size_t)tok * hidden);
    uint4* dst = reinterpret_cast<uint4*>(h + (size_t)b * hidden);
    for (int i = threadIdx.x; i < hidden / 8; i += blockDim.x) dst[i] = __ldg(src + i);

    int before = 0;
    for (int i = threadIdx.x; i < b; i += blockDim.x) before += min(pos[i] / 16 + 1, max_pps);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) before += __shfl_xor_sync(0xffffffffu, before, o);
    if ((threadIdx.x & 31) == 0) s_part[threadIdx.x >> 5] = before;
    __syncthreads();
    int start = 0;
    for (int w = 0; w < 8; ++w) start += s_part[w];
    const int mine = min(pos[b] / 16 + 1, max_pps);
    for (int i = threadIdx.x; i < mine; i += blockDim.x)
        kv_page_indices[start + i] = block_table[(size_t)b * max_pps + i];
    if (threadIdx.x == 0) {
        kv_indptr[b] = start;
        if (b == B - 1) kv_indptr[B] = start + mine;
        kv_last_page_len[b] = pos[b] % 16 + 1;
    }
}

// out = fp16(silu(gate)) * up, the rounding points of the HF MLP (act_fn output is an fp16 tensor).
// gate_up: [rows][2 * inter] (gate columns first); out: [rows][inter].
__global__ void __launch_bounds__(256) silu_mul_kernel(const __half* gate_up, __half* out, int inter, int rows) {
    pdl_begin();
    const int nvec = inter >> 3;
    const long long total = (long long)rows * nvec;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        const int r = (int)(i / nvec), c = (int)(i - (long long)r * nvec);
        const uint4 g = __ldg(reinterpret_cast<const uint4*>(gate_up + (size_t)r * 2 * inter) + c);
        const uint4 u = __ldg(reinterpret_cast<const uint4*>(gate_up + (size_t)r * 2 * inter + inter) + c);
        const __half2* gh = reinterpret_cast<const __half2*>(&g);
        const __half2* uh = reinterpret_cast<const __half2*>(&u);
        uint4 o;
        __half2* oh = reinterpret_cast<__half2*>(&o);
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const float2 f = __half22float2(gh[q]);
            const __half2 act = __floats2half2_rn(f.x / (1.f + __expf(-f.x)), f.y / (1.f + __expf(-f.y)));
            oh[q] = __hmul2(act, uh[q]);
        }
        reinterpret_cast<uint4*>(out + (size_t)r * inter)[c] = o;
    }
}

}  // namespace
}  // namespace leankv

using namespace leankv;

extern "C" int leankv_rmsnorm_f16(void* x, const void* delta, const void* weight, void* y, int n,
                                  float eps, void* stream) {
    if (!x || !weight || !y || n <= 0) return LEANKV_EINVAL;
    if (n % 8 != 0 || !aligned16(x) || !aligned16(weight) || !aligned16(y) || (delta && !aligned16(delta)))
        return LEANKV_EALIGN;
    if (n > kNormThreads * 8 * kNormVecs) return LEANKV_ELIMIT;
    LEANKV_CUDA_TRY(launch_kernel(rmsnorm_kernel, dim3(1), dim3(kNormThreads), 0, static_cast<cudaStream_t>(stream),
                                  static_cast<__half*>(x), static_cast<const __half*>(delta),
                                  static_cast<const __half*>(weight), static_cast<__half*>(y), n, eps));
    return LEANKV_OK;
}

extern "C" int leankv_decode_begin(const void* embed_table, const long long* token, void* h,
                                   int hidden, int vocab, int32_t* state, void* stream) {
    if (!embed_table || !token || !h || !state || hidden <= 0 || vocab <= 0) return LEANKV_EINVAL;
    if (hidden % 8 != 0 || !aligned16(embed_table) || !aligned16(h)) return LEANKV_EALIGN;
    LEANKV_CUDA_TRY(launch_kernel(decode_begin_kernel, dim3(1), dim3(256), 0, static_cast<cudaStream_t>(stream),
                                  static_cast<const __half*>(embed_table), token, static_cast<__half*>(h),
                                  hidden, vocab, state));
    return LEANKV_OK;
}

extern "C" int leankv_rope_f16(const void* qkv, const float* inv_freq, const int32_t* state,
                               void* q_out, void* k_out, int n_q_heads, int n_kv_heads,
                               int head_dim, void* stream) {
    if (!qkv || !inv_freq || !state || !q_out || !k_out || n_q_heads <= 0 || n_kv_heads <= 0)
        return LEANKV_EINVAL;
    if (head_dim != 128) return LEANKV_EUNSUPPORTED;
    LEANKV_CUDA_TRY(launch_kernel(rope_kernel, dim3(n_q_heads + n_kv_heads), dim3(64), 0,
                                  static_cast<cudaStream_t>(stream), static_cast<const __half*>(qkv), inv_freq,
                                  state, static_cast<__half*>(q_out), static_cast<__half*>(k_out), n_q_heads,
                                  n_kv_heads));
    return LEANKV_OK;
}

extern "C" int leankv_decode_end(const void* logits, int vocab, long long* token, long long* history,
                                 int history_cap, int32_t* state, void* stream) {
    if (!logits || !token || !history || !state || vocab <= 0 || history_cap < 0) return LEANKV_EINVAL;
    if (!aligned16(logits)) return LEANKV_EALIGN;
    LEANKV_CUDA_TRY(launch_kernel(decode_end_kernel, dim3(1), dim3(1024), 0, static_cast<cudaStream_t>(stream),
                                  static_cast<const __half*>(logits), vocab, token, history, history_cap,
                                  state + kPos, state + kStep));
    return LEANKV_OK;
}

extern "C" int leankv_decode_end_sharded(const void* logits_local, int vocab_local, int vocab_offset,
                                         long long* token, long long* history, int history_cap, int32_t* state,
                                         const leankv_xchg_t* xchg, int slot, void* stream) {
    if (!logits_local || !token || !history || !state || !xchg || vocab_local <= 0 || vocab_offset < 0 ||
        history_cap < 0)
        return LEANKV_EINVAL;
    if (vocab_local % 8 != 0 || !aligned16(logits_local)) return LEANKV_EALIGN;
    if (xchg->world < 1 || xchg->world > LEANKV_MAX_RANKS || xchg->rank < 0 || xchg->rank >= xchg->world ||
        slot < 0 || slot >= xchg->n_slots || 2 * xchg->world > xchg->world * xchg->max_cols || !xchg->epoch ||
        !xchg->status || xchg->max_wait_iters < 1)
        return LEANKV_EINVAL;
    ShardedEndParams p{};
    p.logits = static_cast<const __half*>(logits_local);
    p.vocab_local = vocab_local;
    p.vocab_offset = vocab_offset;
    p.token = token;
    p.history = history;
    p.history_cap = history_cap;
    p.pos = state + kPos;
    p.step_ptr = state + kStep;
    p.world = xchg->world;
    p.rank = xchg->rank;
    p.limit = xchg->max_wait_iters;
    for (int r = 0; r < xchg->world; ++r) {
        if (!xchg->recv[r] || (reinterpret_cast<uintptr_t>(xchg->recv[r]) & 7u) != 0) return LEANKV_EINVAL;
        p.recv[r] = static_cast<unsigned long long*>(xchg->recv[r]) + (size_t)slot * xchg->world * xchg->max_cols;
    }
    p.epoch = const_cast<int*>(xchg->epoch);
    p.status = xchg->status;
    LEANKV_CUDA_TRY(launch_kernel(decode_end_sharded_kernel, dim3(1), dim3(1024), 0,
                                  static_cast<cudaStream_t>(stream), p));
    return LEANKV_OK;
}

extern "C" int leankv_rmsnorm_rows_f16(void* x, const void* delta, const void* weight, void* y, int rows, int n,
                                       float eps, void* stream) {
    if (!x || !weight || !y || n <= 0 || rows <= 0) return LEANKV_EINVAL;
    if (n % 8 != 0 || !aligned16(x) || !aligned16(weight) || !aligned16(y) || (delta && !aligned16(delta)))
        return LEANKV_EALIGN;
    if (n > kNormThreads * 8 * kNormVecs) return LEANKV_ELIMIT;
    LEANKV_CUDA_TRY(launch_kernel(rmsnorm_kernel, dim3(rows), dim3(kNormThreads), 0,
                                  static_cast<cudaStream_t>(stream), static_cast<__half*>(x),
                                  static_cast<const __half*>(delta), static_cast<const __half*>(weight),
                                  static_cast<__half*>(y), n, eps));
    return LEANKV_OK;
}

extern "C" int leankv_batch_decode_begin(const void* embed_table, const long long* tokens, void* h, int hidden,
                                         int vocab, int B, const int32_t* pos, const int32_t* block_table,
                                         int max_pages_per_seq, int32_t* kv_indptr, int32_t* kv_page_indices,
                                         int32_t* kv_last_page_len, void* stream) {
    if (!embed_table || !tokens || !h || !pos || !block_table || !kv_indptr || !kv_page_indices ||
        !kv_last_page_len || hidden <= 0 || vocab <= 0 || B <= 0 || max_pages_per_seq <= 0)
        return LEANKV_EINVAL;
    if (hidden % 8 != 0 || !aligned16(embed_table) || !aligned16(h)) return LEANKV_EALIGN;
    LEANKV_CUDA_TRY(launch_kernel(batch_begin_kernel, dim3(B), dim3(256), 0, static_cast<cudaStream_t>(stream),
                                  static_cast<const __half*>(embed_table), tokens, static_cast<__half*>(h), hidden,
                                  vocab, B, pos, block_table, max_pages_per_seq, kv_indptr, kv_page_indices,
                                  kv_last_page_len));
    return LEANKV_OK;
}

extern "C" int leankv_silu_mul_f16(const void* gate_up, void* out, int rows, int inter, void* stream) {
    if (!gate_up || !out || rows <= 0 || inter <= 0) return LEANKV_EINVAL;
    if (inter % 8 != 0 || !aligned16(gate_up) || !aligned16(out)) return LEANKV_EALIGN;
    const long long total = (long long)rows * (inter / 8);
    const int grid = (int)std::min<long long>((total + 255) / 256, (long long)sm_count() * 8);
    LEANKV_CUDA_TRY(launch_kernel(silu_mul_kernel, dim3(grid), dim3(256), 0, static_cast<cudaStream_t>(stream),
                                  static_cast<const __half*>(gate_up), static_cast<__half*>(out), inter, rows));
    return LEANKV_OK;
}

extern "C" int leankv_batch_decode_end(const void* logits, int vocab, int B, long long* tokens,
                                       long long* history, int history_cap, int32_t* pos, int32_t* steps,
                                       void* stream) {
    if (!logits || !tokens || !history || !pos || !steps || vocab <= 0 || B <= 0 || history_cap < 0)
        return LEANKV_EINVAL;
    if (!aligned16(logits) || vocab % 8 != 0) return LEANKV_EALIGN;
    LEANKV_CUDA_TRY(launch_kernel(decode_end_kernel, dim3(B), dim3(1024), 0, static_cast<cudaStream_t>(stream),
                                  static_cast<const __half*>(logits), vocab, tokens, history, history_cap, pos,
                                  steps));
    return LEANKV_OK;
}

// ---------------------------------------------------------------------------------------------
// Page table of a paged cache kept on the device (replaces the host loops of
// leankv/turboquant/paged_cache.py:96-103 (_allocate_page), :147-164 (page assignment in update) and
// :215-233 (flat metadata for the attention call)).
// ---------------------------------------------------------------------------------------------
namespace leankv {
namespace {

constexpr int kTableThreads = 1024;

// One CTA. Sequence b grows by t_new tokens: it takes the pages it lacks from the top of the free
// stack (sequence 0 first, as the reference's loop does), its length advances, and the flat
// (kv_indptr, kv_page_indices, kv_last_page_len, start_pos) arrays of the append / attention calls are
// rebuilt. If the stack does not hold enough pages nothing changes and status bit 0 is set.
__global__ void __launch_bounds__(kTableThreads) paged_table_step_kernel(
    int t_new, int B, int32_t* seq_len, int32_t* block_table, int pps_cap, int32_t* free_stack, int32_t* free_top,
    int32_t* kv_indptr, int32_t* kv_page_indices, int32_t* kv_last_page_len, int32_t* start_pos, int32_t* status) {
    __shared__ int s_scan[kTableThreads];
    __shared__ int s_fail, s_top;
    pdl_begin();
    const int b = threadIdx.x;
    const int len = b < B ? seq_len[b] : 0;
    const int have = (len + 15) / 16;
    const int want = b < B ? (len + t_new + 15) / 16 : 0;
    const int need = max(want - have, 0);
    // inclusive scans (Hillis-Steele over the CTA) of the pages needed and of the pages held afterwards
    auto scan = [&](int v) -> int {
        s_scan[b] = v;
        __syncthreads();
        for (int o = 1; o < kTableThreads; o <<= 1) {
            const int add = b >= o ? s_scan[b - o] : 0;
            __syncthreads();
            s_scan[b] += add;
            __syncthreads();
        }
        const int incl = s_scan[b];
        __syncthreads();
        return incl;
    };
    const int need_incl = scan(need);
    const int overflow = __syncthreads_or(b < B && want > pps_cap);   // a row of the block table would not hold it
    if (b == kTableThreads - 1) {
        const int total = need_incl, top = *free_top;                 // the last thread's inclusive sum is the total
        const bool fail = total > top || overflow != 0;
        if (total > top) atomicOr(status, 1);
        if (overflow) atomicOr(status, 2);
        if (!fail) *free_top = top - total;
        s_fail = fail ? 1 : 0;
        s_top = top;
    }
    __syncthreads();
    const int top = s_top;
    int new_len = len;
    if (s_fail == 0 && b < B) {
        const int first = need_incl - need;              // pages popped by sequences before this one
        for (int i = 0; i < need; ++i) block_table[(size_t)b * pps_cap + have + i] = free_stack[top - 1 - first - i];
        new_len = len + t_new;
        seq_len[b] = new_len;
    }
    const int pages_now = b < B ? (new_len + 15) / 16 : 0;
    const int pages_incl = scan(pages_now);
    if (b < B) {
        start_pos[b] = len;
        kv_indptr[b + 1] = pages_incl;
        if (b == 0) kv_indptr[0] = 0;
        const int rem = new_len % 16;
        kv_last_page_len[b] = rem > 0 ? rem : 16;        // 0 -> page_size, the reference's convention (:225-226)
    }
    __syncthreads();
    if (b < B) {
        const int off = pages_incl - pages_now;
        for (int i = 0; i < pages_now; ++i) kv_page_indices[off + i] = block_table[(size_t)b * pps_cap + i];
    }
}

}  // namespace
}  // namespace leankv

extern "C" int leankv_paged_table_step(int t_new, int B, int32_t* seq_len, int32_t* block_table,
                                       int max_pages_per_seq, int32_t* free_stack, int32_t* free_top,
                                       int32_t* kv_indptr, int32_t* kv_page_indices, int32_t* kv_last_page_len,
                                       int32_t* start_pos, int32_t* status, void* stream) {
    if (t_new < 0 || B <= 0 || max_pages_per_seq <= 0 || !seq_len || !block_table || !free_stack || !free_top ||
        !kv_indptr || !kv_page_indices || !kv_last_page_len || !start_pos || !status)
        return LEANKV_EINVAL;
    if (B > kTableThreads) return LEANKV_ELIMIT;
    LEANKV_CUDA_TRY(launch_kernel(paged_table_step_kernel, dim3(1), dim3(kTableThreads), 0,
                                  static_cast<cudaStream_t>(stream), t_new, B, seq_len, block_table, max_pages_per_seq,
                                  free_stack, free_top, kv_indptr, kv_page_indices, kv_last_page_len, start_pos,
                                  status));
    return LEANKV_OK;
}
