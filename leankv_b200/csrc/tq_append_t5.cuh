// Multi-token pool append with the rotation on the fifth-generation tensor cores (included by tq_quantize.cu
// inside namespace leankv::{anonymous}, after tq_append_tc.cuh whose contract and band logic it shares).
//
// Same two-step scheme as tq_pool_append_tc_kernel — a fast rotation y ~ Pi_hi u_hi + Pi_hi u_lo + Pi_lo u_hi
// with fp32 accumulation decides every code that is farther than kBand from all decision boundaries, the
// sequential fp32 chain decides the rest — but the fast rotation is three tcgen05.mma products per k-step on a
// tile of 128 tokens: the unit vectors' fp16 halves and Pi's are written to shared memory in the blocked K-major
// layout of umma.cuh, one thread issues the 24 MMAs (M = N = 128, K = 16), the accumulator (128 tokens x 128
// coordinates, fp32) lives in tensor memory and is read back with tcgen05.ld, one token per thread. No
// ldmatrix / mma.sync instruction stream, no fp32 copy of the unit vectors in shared memory: the rare exact
// chain re-derives u from the fp16 input and the stored norm with the same division.
//
// A CTA of 8 warps quantizes tiles of 128 tokens (8 pages, one per warp when packing) of one (sequence, head,
// K|V); CTAs are persistent over a contiguous range of tiles and keep the fp16 copies of Pi in shared memory,
// reloading them only when their range crosses from K to V.

constexpr int kT5Threads = 256;
constexpr int kT5Tokens = umma::kRows;            // 128
constexpr int kT5Pages = kT5Tokens / 16;          // 8
constexpr size_t kT5SmemBytes = 4 * (size_t)umma::kTileBytes + (size_t)kT5Tokens * kCodeStride + 64;

__global__ void __launch_bounds__(kT5Threads, 1) tq_pool_append_t5_kernel(const AppendTcParams tp, int* status) {
    extern __shared__ __align__(1024) unsigned char t5_smem[];
    uint8_t* s_bh = t5_smem;                                    // Pi high halves: [coordinate j][k], blocked
    uint8_t* s_bl = s_bh + umma::kTileBytes;
    uint8_t* s_ah = s_bl + umma::kTileBytes;                    // unit vectors, high halves: [token][k], blocked
    uint8_t* s_al = s_ah + umma::kTileBytes;
    uint8_t* s_code = s_al + umma::kTileBytes;                  // [128][kCodeStride]
    uint64_t* s_bar = reinterpret_cast<uint64_t*>(s_code + (size_t)kT5Tokens * kCodeStride);
    uint32_t* s_tmem = reinterpret_cast<uint32_t*>(s_bar + 1);
    __shared__ float s_norm[kT5Tokens];
    __shared__ uint16_t s_list[kT5Threads / 32][kListCap];      // per warp: (token row << 7 | coordinate) awaiting the exact chain
    __shared__ float s_bounds[8];

    const AppendParams& p = tp.a;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (warp == 0) umma::tmem_alloc(umma::smem_addr(s_tmem));
    if (tid == 0) umma::bar_init(umma::smem_addr(s_bar));
    pdl_begin();
    if (tid < 8) s_bounds[tid] = tid < 7 ? p.bounds[tid] : __int_as_float(0x7f800000);
    umma::fence_before_sync();
    __syncthreads();
    umma::fence_after_sync();
    const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(s_tmem);

    const long long tile_lo = (long long)blockIdx.x * tp.n_tiles / gridDim.x;
    const long long tile_hi = ((long long)blockIdx.x + 1) * tp.n_tiles / gridDim.x;
    const long long per_which = (long long)p.B * p.H * tp.groups;
    int loaded_which = -1;
    unsigned long long n_exact = 0, n_coords = 0;
    uint32_t phase = 0;
    bool failed = false;

    for (long long tile = tile_lo; tile < tile_hi && !failed; ++tile) {
        const int which = (int)(tile / per_which);
        long long r = tile - (long long)which * per_which;
        const int grp = (int)(r % tp.groups);
        r /= tp.groups;
        const int h = (int)(r % p.H), b = (int)(r / p.H);
        const float* Pi = which == 0 ? p.Pi_k : p.Pi_v;

        umma::fence_before_sync();
        __syncthreads();                 // the previous tile's readers of the code tile, TMEM and operands are done
        umma::fence_after_sync();
        if (which != loaded_which) {
            // B[k][n] = Pi[n][k]: rows of Pi as they are, split into fp16 halves
#pragma unroll 4
            for (int i = tid; i < kDim * (kDim / 8); i += kT5Threads) {
                const int n = i / (kDim / 8), k8 = i % (kDim / 8);
                const float4 w0 = __ldg(reinterpret_cast<const float4*>(Pi + (size_t)n * kDim + 8 * k8));
                const float4 w1 = __ldg(reinterpret_cast<const float4*>(Pi + (size_t)n * kDim + 8 * k8) + 1);
                uint32_t hi[4], lo[4];
                split_h2(w0.x, w0.y, hi[0], lo[0]);
                split_h2(w0.z, w0.w, hi[1], lo[1]);
                split_h2(w1.x, w1.y, hi[2], lo[2]);
                split_h2(w1.z, w1.w, hi[3], lo[3]);
                *reinterpret_cast<uint4*>(s_bh + umma::offset(n, k8)) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
                *reinterpret_cast<uint4*>(s_bl + umma::offset(n, k8)) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
            }
            loaded_which = which;
        }

        const int pos0 = p.start_pos[b];
        const int ord0 = pos0 / 16 + kT5Pages * grp;          // first page ordinal of this tile
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
#pragma unroll
            for (int c = 0; c < 8; ++c) {                      // 8 coordinates = one 16-byte piece of the operands
                uint32_t hi[4], lo[4];
#pragma unroll
                for (int e = 0; e < 4; ++e)
                    split_h2(xr[8 * c + 2 * e] / denom, xr[8 * c + 2 * e + 1] / denom, hi[e], lo[e]);
                *reinterpret_cast<uint4*>(s_ah + umma::offset(row, hf * 8 + c)) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
                *reinterpret_cast<uint4*>(s_al + umma::offset(row, hf * 8 + c)) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
            }
        }
        umma::fence_operands();
        umma::fence_before_sync();
        __syncthreads();
        umma::fence_after_sync();

        // ---- fast rotation: y[token][j] = sum_k u[token][k] Pi[j][k], 24 MMAs from one thread ----
        if (tid == 0) {
            const uint32_t ah = umma::smem_addr(s_ah), al = umma::smem_addr(s_al);
            const uint32_t bh = umma::smem_addr(s_bh), bl = umma::smem_addr(s_bl);
#pragma unroll
            for (int ks = 0; ks < kDim / 16; ++ks) {
                const uint32_t off = (uint32_t)ks * 2 * umma::kLbo;
                umma::mma_f16(tmem_base, umma::desc(al + off), umma::desc(bh + off), ks == 0 ? 0u : 1u);
                umma::mma_f16(tmem_base, umma::desc(ah + off), umma::desc(bl + off), 1u);
                umma::mma_f16(tmem_base, umma::desc(ah + off), umma::desc(bh + off), 1u);
            }
            umma::commit(umma::smem_addr(s_bar));
        }
        const bool done = umma::bar_wait(umma::smem_addr(s_bar), phase);
        phase ^= 1u;
        umma::fence_after_sync();
        if (__syncthreads_or(!done)) {
            failed = true;               // the MMAs did not report completion in time: stop, report, free TMEM below
            break;
        }

        // ---- codes; coordinates close to a boundary are queued for the sequential fp32 chain ----
        // warp w reads accumulator lanes 32 (w % 4) .. + 31 (token rows), warps 0-3 coordinates 0-63, 4-7 the rest
        const float b1 = s_bounds[4], b2 = s_bounds[5], b3 = s_bounds[6];       // 0 < b1 < b2 < b3 (s_bounds[3] = 0)
        const int lane0 = 32 * (warp & 3), col_base = (warp >> 2) * 64;
        const int row = lane0 + lane;
        const int row_pos = ord0 * 16 + row;
        const bool row_ok = row_pos >= pos0 && row_pos < pos_end;
        // exact value of one coordinate: y = fma chain over k ascending, u re-derived from the input and the norm
        auto exact_code = [&](int erow, int coord) -> int {
            const float4* pr = reinterpret_cast<const float4*>(Pi + (size_t)coord * kDim);
            const uint4* xs = reinterpret_cast<const uint4*>(src + (size_t)(ord0 * 16 + erow - pos0) * kDim);
            const float denom = s_norm[erow] + 1e-10f;
            float ye = 0.f;
#pragma unroll 4
            for (int k8 = 0; k8 < kDim / 8; ++k8) {
                const uint4 w = __ldg(xs + k8);
                const float4 p0 = __ldg(pr + 2 * k8), p1 = __ldg(pr + 2 * k8 + 1);
                const float2 a = h2_to_f2(w.x), bb = h2_to_f2(w.y), c = h2_to_f2(w.z), d = h2_to_f2(w.w);
                ye = fmaf(p0.x, a.x / denom, ye);
                ye = fmaf(p0.y, a.y / denom, ye);
                ye = fmaf(p0.z, bb.x / denom, ye);
                ye = fmaf(p0.w, bb.y / denom, ye);
                ye = fmaf(p1.x, c.x / denom, ye);
                ye = fmaf(p1.y, c.y / denom, ye);
                ye = fmaf(p1.z, d.x / denom, ye);
                ye = fmaf(p1.w, d.y / denom, ye);
            }
            int code = 0;
#pragma unroll
            for (int q = 0; q < 7; ++q) code += (ye > s_bounds[q]) ? 1 : 0;
            return code;
        };
        uint32_t near[2] = {0u, 0u};                           // bit i of word c: coordinate col_base + 32 c + i is in the band
#pragma unroll
        for (int c = 0; c < 2; ++c) {
            uint32_t yv[32];
            umma::ld32(yv, tmem_base, lane0, col_base + 32 * c);
            uint32_t packed[8];
#pragma unroll
            for (int i = 0; i < 32; ++i) {
                const float y = __uint_as_float(yv[i]);
                const float ay = fabsf(y);
                const int mag = (ay > b1 ? 1 : 0) + (ay > b2 ? 1 : 0) + (ay > b3 ? 1 : 0);
                const uint32_t code = (uint32_t)(y > 0.f ? 4 + mag : 3 - mag);
                const bool nr = ay <= kBand || fabsf(ay - b1) <= kBand || fabsf(ay - b2) <= kBand ||
                                fabsf(ay - b3) <= kBand;
                if (nr && row_ok) near[c] |= 1u << i;
                if ((i & 3) == 0) packed[i >> 2] = code;
                else packed[i >> 2] |= code << (8 * (i & 3));
            }
            uint32_t* dst = reinterpret_cast<uint32_t*>(s_code + (size_t)row * kCodeStride + col_base + 32 * c);
#pragma unroll
            for (int q = 0; q < 8; ++q) dst[q] = packed[q];      // rows are 4-byte aligned (stride 132)
        }
        if (row_ok) n_coords += 64;
        n_exact += __popc(near[0]) + __popc(near[1]);
        // The band coordinates of all lanes are compacted into a queue; whenever it holds 32 of them every
        // lane runs one exact chain. (A tile of all-zero vectors puts every coordinate in the band.)
        if (__any_sync(0xffffffffu, (near[0] | near[1]) != 0u)) {
            int cnt = 0;                                       // warp-uniform
            auto flush = [&](int n_take) {
                __syncwarp();
                if (lane < n_take) {
                    const int ent = s_list[warp][lane];
                    s_code[(size_t)(ent >> 7) * kCodeStride + (ent & 127)] = (uint8_t)exact_code(ent >> 7, ent & 127);
                }
                const int rest = cnt - n_take;                 // < 32
                const uint16_t moved = lane < rest ? s_list[warp][n_take + lane] : (uint16_t)0;
                __syncwarp();
                if (lane < rest) s_list[warp][lane] = moved;
                cnt = rest;
            };
#pragma unroll 1
            for (int idx = 0; idx < 64; ++idx) {
                const bool flag = ((near[idx >> 5] >> (idx & 31)) & 1u) != 0u;
                const unsigned m = __ballot_sync(0xffffffffu, flag);
                if (m == 0u) continue;
                if (flag) s_list[warp][cnt + __popc(m & ((1u << lane) - 1u))] = (uint16_t)((row << 7) | (col_base + idx));
                cnt += __popc(m);
                if (cnt >= 32) flush(32);
            }
            if (cnt > 0) flush(cnt);
        }
        umma::fence_before_sync();
        __syncthreads();                 // every code of the tile is final
        umma::fence_after_sync();

        // ---- this warp's page of the tile: pack its chunk (same words as tq_pool_append_kernel) ----
        const int page_ord = ord0 + warp;
        const int first = max(pos0, page_ord * 16), last = min(pos_end, page_ord * 16 + 16);
        const int nt_valid = last - first;                    // tokens of this launch in the page
        if (nt_valid <= 0) continue;                          // warp-uniform; CTA-wide syncs are at the loop top
        const int slot0 = first - page_ord * 16;
        const int page = p.kv_page_indices[p.kv_indptr[b] + page_ord];
        if (page < 0 || page >= p.n_pages) continue;          // invalid table entry: write nothing
        const uint8_t* code_rows = s_code + (size_t)(16 * warp) * kCodeStride;
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
    if (failed && tid == 0) atomicOr(status, 1);
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
    // tensor memory goes back before the CTA exits, whatever happened above
    umma::fence_before_sync();
    __syncthreads();
    if (warp == 0) umma::tmem_free(tmem_base);
}
