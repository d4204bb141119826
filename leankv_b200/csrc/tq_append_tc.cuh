// Multi-token pool append with the rotation on tensor cores (included by tq_quantize.cu inside
// namespace leankv::{anonymous}).
//
// The arithmetic contract of this file's header still holds bit for bit: a code is defined by the
// sequential fp32 fma chain y_j = fma(Pi[j][k], u[k], y_j), k ascending. Tensor cores cannot run
// that chain, so the rotation is done twice over:
//   1. fast: u and Pi are split into fp16 high and low parts (x = hi + lo, |lo| <= 2^-11 |hi|) and
//      y ~ Pi_hi u_hi + Pi_hi u_lo + Pi_lo u_hi on m16n8k16 MMAs with fp32 accumulation. The result
//      differs from the chain's value by far less than kBand (the dropped lo x lo term, the
//      remainder of the two-part split, fp16 subnormal rounding of the low parts and the
//      accumulation error of 24 MMAs sum to a few 1e-6 for |y| <= 1);
//   2. exact: a coordinate whose fast value lies within kBand of a decision boundary (a few per
//      thousand) is recomputed with the sequential chain from the fp32 unit vector kept in shared
//      memory, and that value decides the code.
// Every other coordinate is farther from all boundaries than the fast path's error, so its code is
// the chain's code. The fp32 kernels above remain the definition; tests compare whole pools.
//
// A CTA of 4 warps quantizes tiles of 64 tokens (4 pages, one per warp) of one (sequence, head,
// K|V); CTAs are persistent over a contiguous range of tiles and keep the fp16 copies of Pi in
// shared memory, reloading them only when their range crosses from K to V.

constexpr int kTcThreads = 128;
constexpr int kTcTokens = 64;
constexpr int kPiStride = 136;            // halves per row (272 bytes): conflict-free 8 x 16-byte ldmatrix rows
constexpr int kUStride = 136;             // floats per row of the unit-vector tile
constexpr float kBand = 1e-4f;
constexpr int kCodeStride = 132;          // bytes per token row of the code tile: 4-byte reads of 8 tokens x 4 quarters hit 32 banks
constexpr int kListCap = 64;              // queue of boundary-band coordinates: flushed whenever it holds a full warp's worth
constexpr size_t kTcSmemBytes = 2 * (size_t)kDim * kPiStride * sizeof(__half) +
                                (size_t)kTcTokens * kUStride * sizeof(float) + (size_t)kTcTokens * kCodeStride;

struct AppendTcParams {
    AppendParams a;
    int groups;                       // 4-page groups per (sequence, head, K|V)
    long long n_tiles;
    unsigned long long* stats;        // [0] += coordinates recomputed exactly, [1] += coordinates quantized (may be null)
};

__device__ __forceinline__ void ldmatrix_x4(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3, uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
                 : "r"(addr));
}
__device__ __forceinline__ void mma_f16_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// hi = fp16(x) for both elements, lo = fp16(x - hi)
__device__ __forceinline__ void split_h2(float x0, float x1, uint32_t& hi, uint32_t& lo) {
    const __half2 h = __floats2half2_rn(x0, x1);
    const float2 hf = __half22float2(h);
    const __half2 l = __floats2half2_rn(x0 - hf.x, x1 - hf.y);
    hi = *reinterpret_cast<const uint32_t*>(&h);
    lo = *reinterpret_cast<const uint32_t*>(&l);
}

__global__ void __launch_bounds__(kTcThreads, 2) tq_pool_append_tc_kernel(const AppendTcParams tp) {
    extern __shared__ __align__(16) unsigned char tc_smem[];
    __half* s_pih = reinterpret_cast<__half*>(tc_smem);
    __half* s_pil = s_pih + kDim * kPiStride;
    float* s_u = reinterpret_cast<float*>(s_pil + kDim * kPiStride);                 // [64][kUStride]
    uint8_t* s_code = reinterpret_cast<uint8_t*>(s_u + kTcTokens * kUStride);        // [64][kCodeStride]
    __shared__ float s_norm[kTcTokens];
    __shared__ uint16_t s_list[kTcThreads / 32][kListCap];      // per warp: (slot << 7 | coordinate) awaiting the exact chain
    __shared__ float s_bounds[8];

    const AppendParams& p = tp.a;
    pdl_begin();
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t = lane & 3;
    if (tid < 8) s_bounds[tid] = tid < 7 ? p.bounds[tid] : __int_as_float(0x7f800000);

    const long long tile_lo = (long long)blockIdx.x * tp.n_tiles / gridDim.x;
    const long long tile_hi = ((long long)blockIdx.x + 1) * tp.n_tiles / gridDim.x;
    const long long per_which = (long long)p.B * p.H * tp.groups;
    int loaded_which = -1;
    unsigned long long n_exact = 0, n_coords = 0;

    for (long long tile = tile_lo; tile < tile_hi; ++tile) {
        const int which = (int)(tile / per_which);
        long long r = tile - (long long)which * per_which;
        const int grp = (int)(r % tp.groups);
        r /= tp.groups;
        const int h = (int)(r % p.H), b = (int)(r / p.H);
        const float* Pi = which == 0 ? p.Pi_k : p.Pi_v;

        __syncthreads();                 // the previous tile's readers of s_u / s_pi* are done
        if (which != loaded_which) {
            for (int i = tid; i < kDim * kDim / 2; i += kTcThreads) {
                const int j = i >> 6, k2 = (i & 63) * 2;
                const float2 v = __ldg(reinterpret_cast<const float2*>(Pi + j * kDim + k2));
                uint32_t hi, lo;
                split_h2(v.x, v.y, hi, lo);
                *reinterpret_cast<uint32_t*>(&s_pih[j * kPiStride + k2]) = hi;
                *reinterpret_cast<uint32_t*>(&s_pil[j * kPiStride + k2]) = lo;
            }
            loaded_which = which;
        }

        const int pos0 = p.start_pos[b];
        const int ord0 = pos0 / 16 + 4 * grp;                 // first page ordinal of this tile
        const int pos_end = pos0 + p.T_new;
        const __half* src = (which == 0 ? p.k : p.v) + ((size_t)b * p.H + h) * (size_t)p.T_new * kDim;

        // ---- norms and unit vectors: two threads per token, 64 coordinates each ----
        {
            const int row = tid >> 1, hf = tid & 1;
            const int pos = ord0 * 16 + row;
            const bool ok = pos >= pos0 && pos < pos_end;
            float xr[64];
            if (ok) {
                const uint4* s4 = reinterpret_cast<const uint4*>(src + (size_t)(pos - pos0) * kDim + hf * 64);
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
            const double other = __shfl_xor_sync(0xffffffffu, mine, 1);
            const double tot = hf == 0 ? mine + other : other + mine;
            const float norm = (float)sqrt(tot);
            const float denom = norm + 1e-10f;
            if (hf == 0) s_norm[row] = norm;
            float4* dst = reinterpret_cast<float4*>(&s_u[row * kUStride + hf * 64]);
#pragma unroll
            for (int i = 0; i < 16; ++i)
                dst[i] = make_float4(xr[4 * i] / denom, xr[4 * i + 1] / denom, xr[4 * i + 2] / denom, xr[4 * i + 3] / denom);
        }
        __syncthreads();

        // ---- this warp's page ----
        const int page_ord = ord0 + warp;
        const int first = max(pos0, page_ord * 16), last = min(pos_end, page_ord * 16 + 16);
        const int nt_valid = last - first;                    // tokens of this launch in the page
        if (nt_valid <= 0) continue;                          // warp-uniform; CTA-wide syncs are at the loop top
        const int slot0 = first - page_ord * 16;
        const int page = p.kv_page_indices[p.kv_indptr[b] + page_ord];
        const bool page_ok = page >= 0 && page < p.n_pages;

        // ---- fast rotation on tensor cores: rows = the page's 16 token slots, columns = coordinates ----
        float acc[16][4];
#pragma unroll
        for (int n = 0; n < 16; ++n) acc[n][0] = acc[n][1] = acc[n][2] = acc[n][3] = 0.f;
        const float* u_lo_row = &s_u[(16 * warp + g) * kUStride];
        const float* u_hi_row = u_lo_row + 8 * kUStride;
        const uint32_t pi_addr = (uint32_t)__cvta_generic_to_shared((lane < 16 ? s_pih : s_pil)) +
                                 (uint32_t)(((lane & 7) * kPiStride + ((lane >> 3) & 1) * 8) * sizeof(__half));
#pragma unroll 1
        for (int ks = 0; ks < 8; ++ks) {
            uint32_t ah[4], al[4];
            {
                const float2 v0 = *reinterpret_cast<const float2*>(u_lo_row + ks * 16 + 2 * t);
                const float2 v1 = *reinterpret_cast<const float2*>(u_hi_row + ks * 16 + 2 * t);
                const float2 v2 = *reinterpret_cast<const float2*>(u_lo_row + ks * 16 + 8 + 2 * t);
                const float2 v3 = *reinterpret_cast<const float2*>(u_hi_row + ks * 16 + 8 + 2 * t);
                split_h2(v0.x, v0.y, ah[0], al[0]);
                split_h2(v1.x, v1.y, ah[1], al[1]);
                split_h2(v2.x, v2.y, ah[2], al[2]);
                split_h2(v3.x, v3.y, ah[3], al[3]);
            }
#pragma unroll
            for (int n = 0; n < 16; ++n) {
                uint32_t bh0, bh1, bl0, bl1;
                ldmatrix_x4(bh0, bh1, bl0, bl1, pi_addr + (uint32_t)((n * 8 * kPiStride + ks * 16) * sizeof(__half)));
                mma_f16_16816(acc[n], al, bh0, bh1);
                mma_f16_16816(acc[n], ah, bl0, bl1);
                mma_f16_16816(acc[n], ah, bh0, bh1);
            }
        }

        // ---- codes; coordinates close to a boundary are queued for the sequential fp32 chain ----
        const float b1 = s_bounds[4], b2 = s_bounds[5], b3 = s_bounds[6];       // 0 < b1 < b2 < b3 (s_bounds[3] = 0)
        uint8_t* code_rows = s_code + (size_t)(16 * warp) * kCodeStride;
        // exact value of one coordinate: y = fma chain over k ascending, from the fp32 unit vector
        auto exact_code = [&](int slot, int coord) -> int {
            const float4* pr = reinterpret_cast<const float4*>(Pi + (size_t)coord * kDim);
            const float4* ur = reinterpret_cast<const float4*>(&s_u[(16 * warp + slot) * kUStride]);
            float4 pv[kDim / 4];
#pragma unroll
            for (int k4 = 0; k4 < kDim / 4; ++k4) pv[k4] = __ldg(pr + k4);      // one round trip for the whole row
            float ye = 0.f;
#pragma unroll
            for (int k4 = 0; k4 < kDim / 4; ++k4) {
                const float4 uv = ur[k4];
                ye = fmaf(pv[k4].x, uv.x, ye);
                ye = fmaf(pv[k4].y, uv.y, ye);
                ye = fmaf(pv[k4].z, uv.z, ye);
                ye = fmaf(pv[k4].w, uv.w, ye);
            }
            int code = 0;
#pragma unroll
            for (int q = 0; q < 7; ++q) code += (ye > s_bounds[q]) ? 1 : 0;
            return code;
        };
        uint32_t near_lo = 0, near_hi = 0;                     // bit 4n + i: value (n, i) of this lane is in the band
#pragma unroll
        for (int n = 0; n < 16; ++n) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int slot = g + (i >> 1) * 8;
                const int coord = n * 8 + 2 * t + (i & 1);
                const float y = acc[n][i];
                const float ay = fabsf(y);
                const int mag = (ay > b1 ? 1 : 0) + (ay > b2 ? 1 : 0) + (ay > b3 ? 1 : 0);
                const int code = y > 0.f ? 4 + mag : 3 - mag;
                const bool near = ay <= kBand || fabsf(ay - b1) <= kBand || fabsf(ay - b2) <= kBand ||
                                  fabsf(ay - b3) <= kBand;
                code_rows[slot * kCodeStride + coord] = (uint8_t)code;
                if (near && slot >= slot0 && slot < slot0 + nt_valid) {
                    if (n < 8) near_lo |= 1u << (4 * n + i);
                    else near_hi |= 1u << (4 * (n - 8) + i);
                }
            }
        }
        n_coords += (unsigned long long)nt_valid * 4;          // per lane: 128 coordinates / 32 lanes
        n_exact += __popc(near_lo) + __popc(near_hi);
        // The band coordinates of all lanes are compacted into a queue; whenever it holds 32 of them every
        // lane runs one exact chain. (A page of all-zero vectors puts all 2048 coordinates in the band.)
        if (__any_sync(0xffffffffu, (near_lo | near_hi) != 0u)) {
            int cnt = 0;                                       // warp-uniform
            auto flush = [&](int n_take) {
                __syncwarp();
                if (lane < n_take) {
                    const int ent = s_list[warp][lane];
                    code_rows[(ent >> 7) * kCodeStride + (ent & 127)] = (uint8_t)exact_code(ent >> 7, ent & 127);
                }
                const int rest = cnt - n_take;                 // < 32
                const uint16_t moved = lane < rest ? s_list[warp][n_take + lane] : (uint16_t)0;
                __syncwarp();
                if (lane < rest) s_list[warp][lane] = moved;
                cnt = rest;
            };
#pragma unroll 1
            for (int idx = 0; idx < 64; ++idx) {
                const bool flag = ((idx < 32 ? near_lo >> idx : near_hi >> (idx - 32)) & 1u) != 0u;
                const unsigned m = __ballot_sync(0xffffffffu, flag);
                if (m == 0u) continue;
                if (flag) {
                    const int n = idx >> 2, i = idx & 3;
                    const int slot = g + (i >> 1) * 8, coord = n * 8 + 2 * t + (i & 1);
                    s_list[warp][cnt + __popc(m & ((1u << lane) - 1u))] = (uint16_t)((slot << 7) | coord);
                }
                cnt += __popc(m);
                if (cnt >= 32) flush(32);
            }
            if (cnt > 0) flush(cnt);
        }
        __syncwarp();
        if (!page_ok) continue;                                // invalid table entry: write nothing

        // ---- pack this page's chunk (same words as tq_pool_append_kernel), four codes per shared-memory read ----
        uint8_t* chunk = p.pool + (((size_t)page * 2 + which) * p.H + h) * kChunkBytes;
        uint32_t* words = reinterpret_cast<uint32_t*>(chunk);
        __half* norms = reinterpret_cast<__half*>(chunk + kNormOffsetBytes);
        if (lane >= slot0 && lane < slot0 + nt_valid) norms[lane] = __float2half_rn(s_norm[16 * warp + lane]);
        // squeezes the low nibbles of 4 bytes into 16 bits
        auto pack4 = [](uint32_t v) -> uint32_t {
            const uint32_t t2 = (v | (v >> 4)) & 0x00FF00FFu;
            return (t2 | (t2 >> 8)) & 0xFFFFu;
        };
        for (int w = lane; w < kChunkWords; w += 32) {
            const int kk = w >> 6, ui = w & 63;
            if (which == 0) {
                // unit (slot, quarter t4): codes e = coordinates 32 t4 + e; word kk holds codes 8kk..8kk+7 as
                // nibbles and bit kk of codes 24..31 in the nibbles' spare bits
                const int slot = ui >> 2, t4 = ui & 3;
                if (slot < slot0 || slot >= slot0 + nt_valid) continue;
                const uint32_t* c4 = reinterpret_cast<const uint32_t*>(&code_rows[slot * kCodeStride + 32 * t4]);
                const uint32_t lo = c4[2 * kk] & 0x07070707u, hi = c4[2 * kk + 1] & 0x07070707u;
                const uint32_t s_lo = ((c4[6] >> kk) & 0x01010101u) << 3, s_hi = ((c4[7] >> kk) & 0x01010101u) << 3;
                words[w] = pack4(lo) | (pack4(hi) << 16) | pack4(s_lo) | (pack4(s_hi) << 16);
            } else {
                // unit (pair pr, group gg): coordinates 16 gg .. +15 of slots 2 pr (low nibbles) and 2 pr + 1
                const int pr = ui < 32 ? (ui & 3) : 4 + (ui & 3);
                const int gg = (ui & 31) >> 2;
                const int sa = 2 * pr, sb = sa + 1;
                const bool has_a = sa >= slot0 && sa < slot0 + nt_valid, has_b = sb >= slot0 && sb < slot0 + nt_valid;
                if (!has_a && !has_b) continue;
                const uint32_t* ca = reinterpret_cast<const uint32_t*>(&code_rows[sa * kCodeStride + 16 * gg]);
                const uint32_t* cb = reinterpret_cast<const uint32_t*>(&code_rows[sb * kCodeStride + 16 * gg]);
                uint32_t bits = 0;
                if (has_a) bits |= (ca[kk] & 0x07070707u) | (((ca[3] >> kk) & 0x01010101u) << 3);
                if (has_b) bits |= ((cb[kk] & 0x07070707u) << 4) | (((cb[3] >> kk) & 0x01010101u) << 7);
                if (!(has_a && has_b)) {
                    // the other token of the pair was (or will be) written by another launch
                    const uint32_t keep = has_a ? 0xF0F0F0F0u : 0x0F0F0F0Fu;
                    bits |= words[w] & keep;
                }
                words[w] = bits;
            }
        }
    }
    if (tp.stats != nullptr) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            n_exact += __shfl_xor_sync(0xffffffffu, n_exact, o);
            n_coords += __shfl_xor_sync(0xffffffffu, n_coords, o);
        }
        if (lane == 0 && n_coords != 0) {
            atomicAdd(tp.stats, n_exact);
            atomicAdd(tp.stats + 1, n_coords);
        }
    }
}
