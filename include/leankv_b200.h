/*
 * leankv_b200 — C ABI of the B200 (sm_100a) kernels behind the leankv hot paths.
 *
 * The reference project (asmit383/leankv) is pure Python and has no FFI of its own;
 * each entry point below names the reference function whose arithmetic it replaces
 * (paths are relative to the reference project root).
 *
 * Conventions
 *  - every pointer is a DEVICE pointer unless its comment says "host";
 *  - the caller owns all buffers; no entry point allocates, frees or synchronises;
 *  - `stream` is a cudaStream_t passed as void* (NULL = default stream); work is
 *    stream-ordered, entry points may be captured into a CUDA graph;
 *  - return value: 0 on success, a negative LEANKV_E* code otherwise
 *    (leankv_strerror gives the text). Arguments are validated before any launch;
 *  - "workspace" buffers hold split-K partial sums and arrival counters. A workspace
 *    must be zero-filled once after allocation; kernels leave the counters zeroed
 *    on exit. One workspace must not be shared by launches that can overlap in time.
 *    The GEMV entry points keep their counters in the first 16 KiB whatever the shape, so
 *    one workspace (sized for the largest shape) may serve launches of different shapes
 *    with N <= 1 048 576 one after the other.
 */
#ifndef LEANKV_B200_H
#define LEANKV_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define LEANKV_OK 0
#define LEANKV_EINVAL (-1)      /* bad shape / size / null pointer            */
#define LEANKV_EALIGN (-2)      /* pointer or leading dimension misaligned    */
#define LEANKV_EWORKSPACE (-3)  /* workspace too small                        */
#define LEANKV_ECUDA (-4)       /* a CUDA runtime call failed                 */
#define LEANKV_EUNSUPPORTED (-5)/* valid request the kernels do not implement */
#define LEANKV_ELIMIT (-6)      /* size beyond a compiled-in maximum          */

const char* leankv_strerror(int code);
/* ABI version: bumped when a signature changes. */
int leankv_abi_version(void);
/* Text of the last CUDA error seen by this library on the calling thread. */
const char* leankv_last_cuda_error(void);

/* ------------------------------------------------------------------------- *
 * TEAL activation-sparse GEMV (batch 1).
 * Replaces leankv/teal/kernels/sparse_gemv.py:143-181 (sparse_gemv) and the Triton
 * kernel at :61-87; mask semantics follow leankv/teal/sparse_fns.py:32-39:
 *     y[n] = sum over z with |x[z]| > fp16(threshold) of Wt[z][n] * x[z]
 * Wt is the layout produced by prepare_weight_for_sparse_gemv (:229-234):
 * row z holds the N weights that multiply input channel z, rows contiguous.
 * Accumulation is fp32 in a fixed order (results are bit-reproducible run to run);
 * y is rounded to fp16 once.
 * ------------------------------------------------------------------------- */

/* Segments let one launch serve several projections that share x but carry their
 * own thresholds (q/k/v): segment s covers output columns [seg_end[s-1], seg_end[s]).
 * Every seg_end must be a multiple of 256 except the last, which must equal N. */
#define LEANKV_MAX_SEGMENTS 4
typedef struct {
    int   n_segments;                       /* 1..LEANKV_MAX_SEGMENTS */
    int   seg_end[LEANKV_MAX_SEGMENTS];
    float threshold[LEANKV_MAX_SEGMENTS];
} leankv_segments_t;

size_t leankv_sparse_gemv_workspace_bytes(int N, int Z);

/* N % 8 == 0; Wt and y 16-byte aligned. bias / residual may be NULL; when given they are
 * fp16 [N] and are added in fp16 after y has been rounded (bias first, as
 * patching.py:174-175 does, then residual + y as the decoder block does).
 * active_elems (may be NULL) is a uint64 counter that receives += the number of weight
 * elements streamed (channels that passed the threshold x columns); 2 bytes each.
 * Besides those, every CTA asks up to 32 KB of its weight rows into L2 before the previous kernel in the
 * stream has finished (LEANKV_GEMV_PREFETCH_KB, 0 = off): a hint that changes DRAM traffic (about the masked
 * share of those bytes is read for nothing) and timing, never results — L2 is the point of coherence, so
 * even a Wt written by that previous kernel is read correctly afterwards. */
int leankv_sparse_gemv_f16(const void* Wt, const void* x, void* y, int N, int Z,
                           float threshold, const void* bias, const void* residual,
                           void* workspace, size_t workspace_bytes,
                           unsigned long long* active_elems, void* stream);

int leankv_sparse_gemv_seg_f16(const void* Wt, const void* x, void* y, int N, int Z,
                               const leankv_segments_t* segs /* host */,
                               const void* bias, const void* residual,
                               void* workspace, size_t workspace_bytes,
                               unsigned long long* active_elems, void* stream);

/* The two kernels above with the block's RMSNorm fused in front (no reference counterpart: HF runs
 * MistralRMSNorm as separate ops before the patched projections): h is the un-normalised row and
 *   x[z] = norm_weight[z] * fp16( h[z] * rsqrt(mean(h^2) + eps) )
 * is formed on the fly by every CTA (Z % 8 == 0, h 16-byte aligned). Every CTA reads all of h while
 * others may already be writing y, so y must not overlap h (LEANKV_EINVAL otherwise); residual may
 * equal y (each output element is read and written by one thread). */
int leankv_sparse_gemv_rmsnorm_f16(const void* Wt, const void* h, const void* norm_weight, float eps,
                                   void* y, int N, int Z, const leankv_segments_t* segs /* host */,
                                   const void* residual, void* workspace, size_t workspace_bytes,
                                   unsigned long long* active_elems, void* stream);
int leankv_sparse_swiglu_rmsnorm_f16(const void* Wt_gate, const void* Wt_up, const void* h,
                                     const void* norm_weight, float eps, void* y, int N, int Z,
                                     float t_gate, float t_up, void* workspace, size_t workspace_bytes,
                                     unsigned long long* active_elems, void* stream);

/* leankv_sparse_gemv_f16 for callers that cannot provide a workspace because they must not
 * allocate device memory: a server whose pool already owns the whole GPU, a plugin host that keeps
 * the allocator to itself, a loop that cannot afford an allocation's device-wide synchronisation.
 * (No counterpart in the reference, which allocates its output and zeroes it on every call.)
 * The split-K scratch is a fixed 768 KiB array inside the library image; every GPU that loads the
 * library holds it until the process exits. This call allocates and frees nothing.
 *  - Limits: N, Z <= LEANKV_STATIC_GEMV_MAX_DIM and the plan's scratch need <= 768 KiB, otherwise
 *    LEANKV_ELIMIT; no bias / residual / counters.
 *  - The first call on each device looks up the array's device address (that device must be
 *    current, as for any call). Make that first call before starting a stream capture.
 *  - All calls on a device share the one array: calls that can overlap on the GPU (different
 *    streams, or graphs replayed concurrently) race on it and give wrong sums. The part of the array
 *    that must start at zero is cleared on `stream` by each call. */
#define LEANKV_STATIC_GEMV_MAX_DIM 65536
int leankv_sparse_gemv_f16_static(const void* Wt, const void* x, void* y, int N, int Z,
                                  float threshold, void* stream);

/* Fused gate/up SwiGLU: y[n] = silu(Wg.x_g)[n] * (Wu.x_u)[n], where x_g / x_u are x
 * masked with t_gate / t_up (the reference installs separate thresholds on gate_proj
 * and up_proj, leankv/teal/patching.py:101-125). Replaces two sparse_gemv calls plus
 * the act_fn(gate)*up elementwise of the HF MLP. Rounding follows that path: gate and
 * up are rounded to fp16, silu is evaluated in fp32 and rounded to fp16, the product
 * is rounded to fp16. */
size_t leankv_sparse_swiglu_workspace_bytes(int N, int Z);
int leankv_sparse_swiglu_f16(const void* Wt_gate, const void* Wt_up, const void* x,
                             void* y, int N, int Z, float t_gate, float t_up,
                             void* workspace, size_t workspace_bytes,
                             unsigned long long* active_elems, void* stream);

/* ------------------------------------------------------------------------- *
 * TurboQuant (MSE variant, Algorithm 1), reference-format tensors.
 * Replaces leankv/turboquant/quantizer.py:119-129 (quantize) and :131-137
 * (dequantize) with _pack_indices/_unpack_indices (:38-85).
 *   norm = ||x||_2 ; u = x / (norm + 1e-10) ; y = Pi u (fp32 FMA, ascending index) ;
 *   code = number of decision boundaries strictly below y ; codes bit-packed
 * indices: uint8 [n_vec][packed_len(dim,bits)], bits 1 -> 8 per byte, 2 -> 4 per
 * byte, 3..4 -> two nibbles per byte (low nibble = even coordinate). norms fp32.
 * Pi is row-major [dim][dim] fp32 (y = Pi u, i.e. rotate_forward of rotation.py:45-47).
 * dim must be 128, bits 1..4. x_dtype: 0 = fp16, 1 = fp32; rows of x contiguous.
 * ------------------------------------------------------------------------- */
int leankv_tq_packed_len(int dim, int bits);
int leankv_tq_quantize(const void* x, int x_dtype, long long n_vec, int dim, int bits,
                       const float* Pi, const float* decision_boundaries /* 2^bits-1 */,
                       uint8_t* indices, float* norms, void* stream);
/* x_hat[v] = norms[v] * (centroids[codes[v]] @ Pi)   (rotate_backward, rotation.py:50-52) */
int leankv_tq_dequantize(const uint8_t* indices, const float* norms, long long n_vec,
                         int dim, int bits, const float* Pi, const float* centroids,
                         void* x_hat, int out_dtype /* 0 = fp16, 1 = fp32 */, void* stream);

/* ------------------------------------------------------------------------- *
 * Paged 3-bit TurboQuant KV pool (dim 128, 3 bits, 16 tokens per page).
 * The pool replaces the cold store of leankv/turboquant/cache.py:73-76 and borrows
 * the page-table conventions of leankv/turboquant/paged_cache.py:215-233
 * (kv_indptr / kv_page_indices / kv_last_page_len, int32).
 *
 * One layer's pool is [n_pages][2 (K,V)][n_kv_heads][LEANKV_TQ_CHUNK_BYTES] bytes.
 * A chunk holds the 16 tokens of one page for one head: 768 bytes of 3-bit codes
 * (192 words, kernel-native order, see leankv_tq_pool_unpack) followed by 16 fp16 norms.
 * ------------------------------------------------------------------------- */
#define LEANKV_TQ_PAGE_TOKENS 16
#define LEANKV_TQ_DIM 128
#define LEANKV_TQ_CHUNK_BYTES 800

size_t leankv_tq_pool_bytes(int n_pages, int n_kv_heads);

/* Fused rotate + Lloyd-Max quantize + 3-bit pack on append (cache.py:136-142 followed
 * by the torch.cat of :145-159). k, v: fp16 [B][n_kv_heads][T_new][128] contiguous.
 * Token t of sequence b lands at position start_pos[b] + t of that sequence; its page
 * is kv_page_indices[kv_indptr[b] + pos / 16]. Pages must already be assigned.
 * start_pos: int32 [B] device. */
int leankv_tq_pool_append(const void* k, const void* v, int B, int n_kv_heads, int T_new,
                          const float* Pi_k, const float* Pi_v,
                          const float* decision_boundaries /* 7 */,
                          void* pool, int n_pages,
                          const int32_t* kv_indptr, const int32_t* kv_page_indices,
                          const int32_t* start_pos, void* stream);

/* Appends of 16 or more tokens per sequence (prompt processing, where the reference quantizes the
 * flushed tokens with one dense fp32 matmul, cache.py:136-142 / quantizer.py:119-129) run the
 * rotation on tensor cores and re-derive every coordinate that lands within 1e-4 of a decision
 * boundary with the sequential fp32 chain, so the codes are those of the definition above.
 * stats[0] = coordinates re-derived, stats[1] = coordinates quantized on the current device since
 * the last reset (synchronous copy; reset != 0 clears the counters). */
int leankv_tq_band_stats(unsigned long long* stats /* host, 2 */, int reset);
/* *status = 0 unless a bounded wait for the tensor cores inside a multi-token append has ever run out on the
 * current device (the pages written by that launch are then incomplete). Synchronous copy. */
int leankv_tq_append_status(int* status /* host */);

/* Pool -> reference format for pages of one sequence: codes as nibble-packed uint8
 * [n_kv_heads][n_tokens][64] and norms fp32 [n_kv_heads][n_tokens] (the fp16 pool
 * norm widened), for K (which = 0) or V (which = 1). */
int leankv_tq_pool_unpack(const void* pool, int n_pages, int n_kv_heads,
                          const int32_t* page_indices /* device, ceil(n_tokens/16) */,
                          int n_tokens, int which, uint8_t* indices, float* norms,
                          void* stream);

/* Decode attention straight from the packed pool: for each sequence b and query head h
 *   out[b][h] = softmax_t( scale * q[b][h] . k_hat[b][kvh][t] ) . v_hat[b][kvh][t]
 * with k_hat / v_hat the TurboQuant reconstructions (quantizer.py:131-137) that
 * cache.py:169-189 would materialise; they are never formed: the query is rotated once,
 * scores and the value sum are taken in rotated space on tensor cores, and the output is
 * rotated back once. q, out: fp16 [B][n_q_heads][128]. n_q_heads / n_kv_heads must be 4
 * (GQA-4) in this version. kv_indptr is a prefix sum (non-decreasing); kv_last_page_len[b] in
 * 1..16; a sequence with kv_indptr[b+1] == kv_indptr[b] yields zeros. max_pages_per_seq sizes
 * the grid and the workspace (host value, >= the longest sequence's page count). centroids is read on the
 * host (the codebook is a compile-time-like constant of the cache): it is turned into
 * register look-up tables that travel as kernel arguments. The first 4 bytes of the
 * workspace are a status word (see leankv_tq_decode_attn_status). The workspace must be zeroed
 * before its first use; calls of one shape (B, heads, max_pages_per_seq) may then share it for
 * ever (the arrival counters reset themselves). Its layout depends on the shape, so a workspace
 * that has served another shape must be zeroed again (all but the status word) before it serves
 * this one. */
size_t leankv_tq_decode_attn_workspace_bytes(int B, int n_q_heads, int n_kv_heads,
                                             int max_pages_per_seq);
int leankv_tq_decode_attn(const void* q, void* out, int B, int n_q_heads, int n_kv_heads,
                          const void* pool, int n_pages,
                          const int32_t* kv_indptr, const int32_t* kv_page_indices,
                          const int32_t* kv_last_page_len, int max_pages_per_seq,
                          const float* Pi_k, const float* Pi_v,
                          const float* centroids /* host, 8 */, float scale,
                          void* workspace, size_t workspace_bytes, void* stream);

/* Same attention for a caller that already holds the rotated query q_rot = Pi_k q
 * (fp32 [B][n_q_heads][128], e.g. from leankv_decode_qkv_post): skips the query-rotation
 * launch. Everything else as leankv_tq_decode_attn.
 * flags: 0, or LEANKV_ATTN_EARLY_FETCH. With the flag the kernel starts reading the page table
 * and fetching every page except each sequence's last one while the launch queued directly
 * before it may still be running (programmatic dependent launch); q_rot and the last pages are
 * read only after that launch has completed. The flag is therefore only correct when the
 * preceding launch writes nothing but q_rot and the last page of each sequence, which is what
 * leankv_decode_qkv_post / leankv_batch_qkv_post do (the decode loops pass the flag). Without
 * it the call has plain stream-order semantics after any launch, e.g. a multi-page
 * leankv_tq_pool_append. */
#define LEANKV_ATTN_EARLY_FETCH 1
int leankv_tq_decode_attn_rotated(const float* q_rot, void* out, int B, int n_q_heads, int n_kv_heads,
                                  const void* pool, int n_pages,
                                  const int32_t* kv_indptr, const int32_t* kv_page_indices,
                                  const int32_t* kv_last_page_len, int max_pages_per_seq,
                                  const float* Pi_v, const float* centroids /* host, 8 */, float scale,
                                  void* workspace, size_t workspace_bytes, int flags, void* stream);

/* Device status word of the bounded waits inside the attention kernel (0 = no wait
 * ever gave up). Copied to *status with a synchronous 4-byte copy from `workspace`. */
int leankv_tq_decode_attn_status(const void* workspace, int* status /* host */);

/* Causal attention of a chunk of T prompt tokens (absolute positions start_pos .. start_pos+T-1) of ONE
 * sequence over its packed pages — the chunked-prefill counterpart of leankv_tq_decode_attn. The
 * chunk's K/V must already be in the pool (leankv_tq_pool_append before this call), so that, like the
 * reference's TurboQuantCache with hot_buffer_size = 0 (leankv/turboquant/cache.py:84-127: update()
 * returns de-quantized K/V for all tokens, the new ones included), every token attends to quantized
 * keys and values only, and never to an fp16 copy. Replaces, for prompt chunks, cache.update +
 * eager attention (leankv/turboquant/cache.py:136-142, transformers modeling_mistral.py:96-117).
 * q, out: [T][n_q_heads][128] fp16. seq_pages (device): the sequence's page ids in order, at least
 * (start_pos + T + 15) / 16 of them. Three launches: the query rotation (tcgen05 tensor cores, fp16
 * high/low split of Pi_K), the attention kernel (one CTA per 32 query tokens, kv head and page range: a
 * page is de-quantized once per 32 tokens into fp16 operand tiles; scores and the value sum on tensor cores
 * with the query as fp16 high + low halves and fp32 accumulation: tcgen05.mma with the accumulators in
 * tensor memory by default; LEANKV_PREFILL_MMA=sync in the environment selects an mma.sync form, =ws a
 * warp-specialised tcgen05 form with query and probabilities as tensor-memory operands), and the merge of
 * the page ranges with the inverse value rotation. The result agrees with decode steps at the same
 * positions to fp16 rounding (rel-L2 < 5e-4 in the tests). The workspace's first word is the status word
 * and must be zero before the first use (bit 0: a bounded wait ran out, bit 1: a page id out of range;
 * with bit 0, bits 4..6 say which wait: page copy, score MMAs, value MMAs); the rest needs no preparation
 * and one workspace may serve chunks of any length. */
size_t leankv_tq_prefill_attn_workspace_bytes(int T, int start_pos, int n_q_heads, int n_kv_heads);
int leankv_tq_prefill_attn(const void* q, void* out, int T, int start_pos, int n_q_heads, int n_kv_heads,
                           const void* pool, int n_pages, const int32_t* seq_pages, const float* Pi_k,
                           const float* Pi_v, const float* centroids, float scale, void* workspace,
                           size_t workspace_bytes, void* stream);

/* ------------------------------------------------------------------------- *
 * Glue kernels of a batch-1 decode step (no reference counterpart: the reference leaves
 * these steps to the HF modules around its hooks — MistralRMSNorm, apply_rotary_pos_emb,
 * embed_tokens, argmax of generate()). They exist so that a whole decode step, including
 * the position / page-table bookkeeping, can be replayed as one CUDA graph.
 *
 * state: int32[8] on the device:
 *   [0] pos        tokens already cached = position of the token being decoded
 *   [1] step       tokens generated so far (index into history)
 *   [2],[3]        kv_indptr of the single sequence {0, pages in use after this append}
 *   [4]            kv_last_page_len after this append
 *   [5]            start_pos of this append
 * ------------------------------------------------------------------------- */
/* If delta != NULL: x += delta first (fp16 add, written back: the residual stream).
 * Then y = weight * fp16(x * rsqrt(mean(x^2) + eps)); fp16 [n], one vector. */
int leankv_rmsnorm_f16(void* x, const void* delta, const void* weight, void* y, int n, float eps,
                       void* stream);
/* h = embed_table[*token]; state[2..5] derived from state[0]. hidden % 8 == 0. */
int leankv_decode_begin(const void* embed_table, const long long* token, void* h, int hidden,
                        int vocab, int32_t* state, void* stream);
/* Rotary embedding (rotate_half form, position state[0]) of the first n_q_heads + n_kv_heads
 * 128-wide heads of a fused qkv row; inv_freq fp32 [64]. */
int leankv_rope_f16(const void* qkv, const float* inv_freq, const int32_t* state, void* q_out,
                    void* k_out, int n_q_heads, int n_kv_heads, int head_dim, void* stream);
/* leankv_rope_f16 + leankv_tq_pool_append (one token, one sequence) + the query rotation of
 * leankv_tq_decode_attn in a single launch, bit-identical to the three: qkv is the fused
 * projection row [q heads | k heads | v heads] x 128 fp16; the token's position is state[0] and
 * its page is page_indices[state[0] / 16]; q_rot (fp32 [n_q_heads][128]) receives Pi_k rope(q).
 * The rotations are passed TRANSPOSED (Pi_k_t[k][j] = Pi_k[j][k], row-major) for coalesced reads. */
int leankv_decode_qkv_post(const void* qkv, const float* inv_freq, const int32_t* state,
                           const float* Pi_k_t, const float* Pi_v_t, const float* decision_boundaries,
                           void* pool, int n_pages, const int32_t* page_indices,
                           int n_q_heads, int n_kv_heads, float* q_rot, void* stream);
/* *token = argmax(logits) (lowest index on ties); history[state[1]] = *token;
 * state[1] += 1; state[0] += 1. */
int leankv_decode_end(const void* logits, int vocab, long long* token, long long* history,
                      int history_cap, int32_t* state, void* stream);

/* ------------------------------------------------------------------------- *
 * Tensor-parallel row-split projections: GEMV + all-reduce in one kernel.
 * The reference has no multi-GPU path; this is the exchange step of the tensor-parallel
 * decode (one process per GPU). Rank r computes its partial y_r = Wt_r^T . mask(x_r) over
 * its slice of the input channels. Every thread of the CTA that finishes a 256-column tile
 * sends its column's fp32 value, tagged with the step's epoch in the same 64-bit store, into
 * every rank's receive area through peer-mapped pointers (NVLink); it then polls its
 * column's words in the local area until all ranks' values of this epoch are there and adds
 * them in rank order (fp32, rounded once, then + residual). Every rank gets bit-identical y
 * without a separate collective launch, fence or flag.
 *
 * Receive area of a rank: 64-bit words [n_slots][world][max_cols], zeroed once and never
 * reset. Every all-reduce inside one decode step uses its own slot (>= 2 slots per step);
 * *epoch (device word, > 0, same on all ranks) changes between steps (leankv_xchg_advance).
 * A poll gives up after max_wait_iters tries: the kernel then sets *status (device word,
 * sticky: later launches do not poll) and returns normally.
 * ------------------------------------------------------------------------- */
#define LEANKV_MAX_RANKS 8
typedef struct {
    int   world, rank;
    int   n_slots, max_cols;                 /* max_cols % 256 == 0 */
    int   max_wait_iters;
    void* recv[LEANKV_MAX_RANKS];            /* rank r's receive area as mapped in this process */
    const int32_t* epoch;
    int32_t* status;
} leankv_xchg_t;

size_t leankv_xchg_recv_bytes(int world, int n_slots, int max_cols);
/* *epoch += 1 (one thread). */
int leankv_xchg_advance(int32_t* epoch, void* stream);
/* y = residual + fp16( sum over ranks of Wt_r^T . mask_t(x_r) ), see above. */
int leankv_sparse_gemv_allreduce_f16(const void* Wt, const void* x, void* y, int N, int Z,
                                     float threshold, const void* residual,
                                     void* workspace, size_t workspace_bytes,
                                     unsigned long long* active_elems,
                                     const leankv_xchg_t* xchg, int slot, void* stream);
/* leankv_decode_end for an output head split over the vocabulary: logits_local is this rank's slice
 * (vocab_local entries starting at global index vocab_offset; vocab_local % 8 == 0). The ranks exchange
 * their {best value, index} through `slot` of the receive areas (2 words per rank) and all store the same
 * token (largest value, lowest index on ties). Being the last exchange of a step, the call also adds 1 to
 * *xchg->epoch, so a decode step that ends with it needs no leankv_xchg_advance. A bounded wait that runs out
 * sets *xchg->status like the GEMV's. */
int leankv_decode_end_sharded(const void* logits_local, int vocab_local, int vocab_offset, long long* token,
                              long long* history, int history_cap, int32_t* state,
                              const leankv_xchg_t* xchg, int slot, void* stream);
/* Device memory that other processes on this node can map (cudaMalloc + CUDA IPC):
 * alloc returns the pointer and a 64-byte handle to hand to the peers; open maps a peer's
 * handle into this process (enables peer access); close / free undo them. */
int leankv_ipc_alloc(size_t bytes, void** ptr, unsigned char handle[64]);
int leankv_ipc_open(const unsigned char handle[64], void** ptr);
int leankv_ipc_close(void* ptr);
int leankv_ipc_free(void* ptr);

/* ------------------------------------------------------------------------- *
 * Glue kernels of a batched decode step (B sequences, one new token each, dense library
 * GEMMs between them: the reference runs its dense path at batch > 1,
 * leankv/teal/patching.py:155-157, with HF modules around the cache). Like the batch-1
 * set they have no reference counterpart; they keep positions and the page table on the
 * device so that a step replays as one CUDA graph.
 *
 * Sequence b has pos[b] tokens cached and owns the pages block_table[b][0..max_pages_per_seq);
 * each step the flat (kv_indptr, kv_page_indices, kv_last_page_len) triple of
 * leankv/turboquant/paged_cache.py:215-233 is rebuilt from them.
 * ------------------------------------------------------------------------- */
/* RMSNorm of `rows` independent vectors (x, delta, y: fp16 [rows][n]); see leankv_rmsnorm_f16. */
int leankv_rmsnorm_rows_f16(void* x, const void* delta, const void* weight, void* y, int rows, int n,
                            float eps, void* stream);
/* h[b] = embed_table[tokens[b]]; kv_indptr [B+1], kv_page_indices [sum of pages in use],
 * kv_last_page_len [B] for the step that appends one token to every sequence. */
int leankv_batch_decode_begin(const void* embed_table, const long long* tokens, void* h, int hidden,
                              int vocab, int B, const int32_t* pos, const int32_t* block_table,
                              int max_pages_per_seq, int32_t* kv_indptr, int32_t* kv_page_indices,
                              int32_t* kv_last_page_len, void* stream);
/* leankv_decode_qkv_post for B sequences: qkv fp16 [B][(n_q_heads + 2 n_kv_heads) * 128],
 * q_rot fp32 [B][n_q_heads][128]; token of sequence b goes to position pos[b], page
 * kv_page_indices[kv_indptr[b] + pos[b] / 16]. */
int leankv_batch_qkv_post(const void* qkv, int B, const float* inv_freq, const int32_t* pos,
                          const int32_t* kv_indptr, const float* Pi_k_t, const float* Pi_v_t,
                          const float* decision_boundaries, void* pool, int n_pages,
                          const int32_t* kv_page_indices, int n_q_heads, int n_kv_heads,
                          float* q_rot, void* stream);
/* out[r][i] = fp16(silu(gate_up[r][i])) * gate_up[r][inter + i]  (LlamaMLP's act_fn(gate) * up). */
int leankv_silu_mul_f16(const void* gate_up, void* out, int rows, int inter, void* stream);
/* Per sequence: tokens[b] = argmax(logits[b]) (lowest index on ties);
 * history[b][steps[b]] = tokens[b]; steps[b] += 1; pos[b] += 1. vocab % 8 == 0. */
int leankv_batch_decode_end(const void* logits, int vocab, int B, long long* tokens,
                            long long* history, int history_cap, int32_t* pos, int32_t* steps,
                            void* stream);

/* ------------------------------------------------------------------------- *
 * Page table of a paged cache, kept on the device. Replaces the host loops of
 * leankv/turboquant/paged_cache.py: _allocate_page (:96-103, LIFO free list), the page assignment
 * of update (:147-164) and the flat metadata built for every attention call (:215-233).
 *
 * State (int32, device): seq_len [B]; block_table [B][max_pages_per_seq] (pages of sequence b in
 * order); free_stack [n_pages] with *free_top entries in use (the top is popped first).
 * One step: every sequence grows by t_new tokens (t_new = 0 only rebuilds the flat arrays), taking
 * the pages it lacks from the stack, sequence 0 first. Outputs for leankv_tq_pool_append /
 * leankv_tq_decode_attn: kv_indptr [B+1], kv_page_indices [pages in use], kv_last_page_len [B]
 * (16 for a full last page), start_pos [B] (length before this step).
 * If the stack holds too few pages (status |= 1) or a row of the block table would overflow
 * (status |= 2) no sequence grows: the host mirrors the arithmetic and raises before launching,
 * the status word is the backstop. B <= 1024.
 * ------------------------------------------------------------------------- */
int leankv_paged_table_step(int t_new, int B, int32_t* seq_len, int32_t* block_table,
                            int max_pages_per_seq, int32_t* free_stack, int32_t* free_top,
                            int32_t* kv_indptr, int32_t* kv_page_indices, int32_t* kv_last_page_len,
                            int32_t* start_pos, int32_t* status, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* LEANKV_B200_H */
