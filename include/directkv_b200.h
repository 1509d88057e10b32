/*
 * directkv_b200 - C ABI of the B200 (sm_100a) decode-attention engine.
 *
 * This is the drop-in boundary for the reference's extension module
 * (directkv/kernel/smpv2_extension.cu, loaded by directkv/kernel/__init__.py): plain pointers,
 * sizes and a stream handle go in, an int status comes out.  No torch types appear here; the
 * Python package turns tensors into pointers and a non-zero status into RuntimeError, which
 * is what the reference's TORCH_CHECK failures surface as.
 *
 * Conventions
 *  - bf16 everywhere for Q/K/V/X/W/O; head_dim is 128 (directkv/directkv_backend.py:163-169).
 *  - KV pools are [n_slots, nh_kv, 128] bf16, in host-pinned (mapped) memory or in device
 *    memory: the layout of DirectKVTokenToKVPool (directkv/directkv_pool.py:96-130) and, with
 *    slot = row * row_stride + position, of DirectKVRequestPool
 *    (directkv/directkv_request_pool.py:66-76).
 *  - `stream` is a cudaStream_t passed as void*; every call only enqueues work unless said
 *    otherwise.  Pointers must stay valid until that work has run.
 *  - All functions return DKV_OK or an error code; dkv_last_error() gives the text for the
 *    calling thread.
 *  - A context belongs to one device and one host thread at a time (the reference's module is
 *    likewise single-threaded per process: directkv/kernel/smpv2_extension.cu:53-61).
 */
#ifndef DIRECTKV_B200_H
#define DIRECTKV_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define DKV_OK                  0
#define DKV_ERR_INVALID         1   /* bad argument (reference: TORCH_CHECK -> RuntimeError) */
#define DKV_ERR_CUDA            2   /* a CUDA runtime/driver call failed */
#define DKV_ERR_UNSUPPORTED     3   /* shape outside what the kernels handle */
#define DKV_ERR_NOT_REGISTERED  4   /* layer id unknown (reference: "call smpv2_init_tma first") */
#define DKV_ERR_DEVICE_STATUS   5   /* the device status word is non-zero (bounded wait ran out, bad slot) */

/* Bits of the device status word (dkv_read_status). */
#define DKV_STATUS_WAIT_TIMEOUT  (1u << 0)
#define DKV_STATUS_BAD_SLOT      (1u << 1)
#define DKV_STATUS_BAD_POSITION  (1u << 2)
#define DKV_STATUS_TMEM_TIMEOUT  (1u << 3)
#define DKV_STATUS_EXCHANGE_ORDER (1u << 4)  /* dkv_decode_exchange: a record of another step arrived (calls of the ranks do not line up) */
#define DKV_STATUS_BAD_PAGE      (1u << 5)  /* a length or row led outside the page table; the entry was not read */
/* Set together with a timeout bit: the kernel that gave up waiting. */
#define DKV_STATUS_IN_STREAMING  (1u << 8)
#define DKV_STATUS_IN_PROJ_LOAD  (1u << 9)
#define DKV_STATUS_IN_PROJ_MMA   (1u << 10)
#define DKV_STATUS_IN_EXTEND     (1u << 11)
#define DKV_STATUS_IN_EXCHANGE   (1u << 12)

/* How the token decoded in this step enters dkv_decode. */
#define DKV_NEW_NONE     0   /* every attended token is already in the pool */
#define DKV_NEW_PROJECT  1   /* K/V = X . Wk^T / Wv^T on tensor cores, Neox RoPE on K, stored to the pool */
#define DKV_NEW_GIVEN    2   /* caller passes the token's (already rotated) K/V rows */

typedef struct dkv_context dkv_context;

int         dkv_version(void);
const char* dkv_last_error(void);

/* One context per device: owns scratch memory, the status word and the per-layer tables. */
int dkv_context_create(int device, dkv_context** out);
int dkv_context_destroy(dkv_context* ctx);

/*
 * Pre-sizes scratch so that later calls with batch <= max_rows query rows
 * (requests for decode, batch * S_new for dkv_smpv2_fwd), nh_q/nh_kv heads and hidden size
 * allocate nothing (needed before CUDA-graph capture; the reference pre-allocates in
 * smpv2_init_tma, directkv/kernel/smpv2_extension.cu:412-422).
 */
int dkv_context_reserve(dkv_context* ctx, int64_t max_rows, int nh_q, int nh_kv, int hidden);

/* Knobs, by name: "attn_variant" (-1 = automatic, 0..2), "attn_mma" (-1 = automatic: warp-level tensor-core
 * inner product when 2..16 query heads share a KV head of a pool in HBM; 0 = never; 1 = always), "attn_mma8" (1 = query heads on the N
 * side of the tensor-core product when at most 8 share a KV head, default; 0 = always the 16-row form), "extend_rowwise" (0/1),
 * "extend_pingpong" (1 = two query tiles per CTA, default; 0 = first form of the extend kernel), "proj_decode"
 * (-1 = use the decode-batch projection kernel where it can run under the streaming kernel, 0 = never, 1 = for
 * every batch of up to 512 tokens), "proj_gemv" (1 = one or two new tokens going to a pool in device memory are projected by the
 * matrix-vector kernel on the CUDA cores, default; 0 = always a tensor-core kernel), "proj_wide" (0 = 128-token projection tiles only), "attn_ctas" (CTAs of the streaming kernel,
 * 0 = one per SM), "attn_min_units" (pools in device memory: a step with fewer 16-token tiles per warp of the streaming grid than this
 * is a short step - its tiles go to about 70 % of the warps, two or more per warp, dealt out over the CTAs in turn; 1..64, default 5;
 * 1 = never), "check_coresidency" (any value: verifies that a 16-warp streaming CTA and a decode-projection
 * CTA fit one SM together, DKV_ERR_UNSUPPORTED with the register and shared-memory figures otherwise), "attn_self_scan" (1 = batches of up to 32 requests run without the
 * prep launch, the kernels scan the lengths themselves, default; 0 = always launch it), "proj_split_k" (0 = automatic), "profile_attn" (0/1, see dkv_profile_read), "wait_limit_ms" (how long
 * dkv_decode_exchange's consumer kernel waits for its peers before it reports DKV_STATUS_WAIT_TIMEOUT; 2000). */
int dkv_context_set(dkv_context* ctx, const char* key, int value);

/*
 * Profiling counters.  With dkv_context_set(ctx, "profile_attn", 1) every launch of the
 * KV-streaming kernel is bracketed by CUDA events on the stream it is launched on;
 * this call synchronises the device and returns their summed duration, how many launches
 * were bracketed, and how many kernels the context has launched in total since the last reset.
 */
int dkv_profile_read(dkv_context* ctx, double* attn_ms_total, long long* attn_launches, long long* total_launches,
                     int reset);

/* Blocks until the stream work touching the status word is done is NOT implied: this
 * synchronises the device, copies the status word and optionally clears it. */
int dkv_read_status(dkv_context* ctx, unsigned int* status, int clear);

/*
 * Per-layer registration: replaces smpv2_init_tma(layer_id, X_max, Wk, Wv, Q_max, K_max, V_max)
 * (directkv/kernel/smpv2_extension.cu:363-423).  Builds and caches the TMA descriptors of the
 * KV pool and of the projection weights.  Pointers must stay valid while the layer is
 * registered.  wk/wv/cos_sin may be NULL for an attention-only layer.
 */
typedef struct {
    void*        k_pool;      /* [n_slots, nh_kv, 128] bf16; host-pinned or device */
    void*        v_pool;
    int64_t      n_slots;
    int          nh_kv;
    int          page_size;   /* tokens per page, power of two >= 1 (paged calls) */
    int64_t      row_stride;  /* slots per pool row (calls with page_table == NULL) */
    const void*  wk;          /* [nh_kv, 128, hidden] bf16, device */
    const void*  wv;
    int          hidden;      /* multiple of 64 */
    const float* cos_sin;     /* [max_pos, 128] fp32 = [cos | sin], device; NULL = no RoPE (OPT) */
    int          max_pos;
} dkv_layer_desc;

int dkv_layer_register(dkv_context* ctx, int layer_id, const dkv_layer_desc* desc);
int dkv_layer_unregister(dkv_context* ctx, int layer_id);

/*
 * One decode step of one layer for a ragged batch: replaces the kernel path of
 * DirectKVBackend.forward_decode (directkv/directkv_backend.py:527-627) and, for every length,
 * its torch path _sdpa_decode_directkv (:781-825) / _sdpa_decode_manual (:835-859).
 *
 * Token t of request b lives at slot
 *     page_table[row(b), t / page_size] * page_size + t % page_size        (paged)
 *     row(b) * row_stride + t                                              (page_table == NULL)
 * with row(b) = row_map ? row_map[b] : b.  seq_lens[b] counts the tokens attended, including
 * the token decoded now unless new_mode == DKV_NEW_NONE.  All index arrays are int32 in
 * device memory and are read on the device, so the call can be captured in a CUDA graph and
 * replayed with new lengths.
 */
typedef struct {
    int            layer_id;
    int            batch;
    int            nh_q;
    const void*    q;            /* bf16 device, row b at q + b * q_stride elements, [nh_q, 128] */
    int64_t        q_stride;
    void*          out;          /* bf16 device, row b at out + b * out_stride; may be NULL */
    int64_t        out_stride;
    const int32_t* seq_lens;     /* [batch] */
    const int32_t* page_table;   /* [rows, pt_stride] or NULL */
    int            pt_stride;
    const int32_t* row_map;      /* [batch] or NULL */
    int            new_mode;     /* DKV_NEW_* */
    const void*    x;            /* [batch, hidden] bf16 device (DKV_NEW_PROJECT) */
    const void*    k_new;        /* [batch, nh_kv, 128] bf16 device (DKV_NEW_GIVEN) */
    const void*    v_new;
    int            save_kv_cache;/* store the new token's K/V to the pool */
    float          softmax_scale;
    float*         lse_out;      /* [batch, nh_q] natural-log LSE, or NULL */
    float*         partial_out;  /* [batch, nh_q, 132] unnormalised (O[128], m_log2, l, pad) or NULL */
    const int32_t* pos_offset;   /* [batch] or NULL: added to seq_lens[b] - 1 to get the new token's absolute
                                    (RoPE) position when this pool holds only a later part of the sequence */
    /* Attend a COPY of the past rows instead of the layer's own pool (0 / NULL: off).  kv_source_layer is another
     * registered layer - typically rows that the copy engines brought from the host pool into HBM, which reach
     * the full rate of the host link where reads issued by the SMs reach 0.92 of it - addressed by
     * src_page_table / src_pt_stride (its page size) or src_row_map (its row_stride).  The new token is still
     * projected with, positioned by and stored to `layer_id` through page_table / row_map above. */
    int            kv_source_layer;
    const int32_t* src_page_table;
    int            src_pt_stride;
    const int32_t* src_row_map;
    int            pt_rows;      /* rows of page_table, or 0 when unknown: with it, a row_map entry beyond the table is
                                    reported (DKV_STATUS_BAD_PAGE) instead of read; page indices are always held
                                    below pt_stride */
} dkv_decode_args;

int dkv_decode(dkv_context* ctx, const dkv_decode_args* args, void* stream);

/* Combines nranks sets of unnormalised partials [nranks, rows, 132] (sequence split across
 * GPUs, after the all-gather) into bf16 out [rows, 128] and optional lse [rows]. */
int dkv_merge_partials(dkv_context* ctx, const float* parts, int nranks, int64_t rows, void* out, float* lse,
                       void* stream);

/*
 * Sequence split with the exchange fused into the kernels (no collective call).  Each rank creates an
 * exchange, passes its 64-byte handle to the other ranks of the box (any side channel), and connects to
 * theirs.  dkv_decode_exchange then runs the rank's part of the decode: its merge kernel stores the
 * unnormalised (O, m, l) record of every (request, head) row straight into every rank's exchange buffer -
 * plain stores over NVLink for peers - and bumps a per-source arrival counter there; a second kernel waits
 * (bounded) until all sources have delivered and merges from this GPU's own memory into out [batch, nh_q,
 * 128] bf16 (and lse).  All ranks must call it the same number of times with the same batch * nh_q.
 * No counterpart in the reference (which is single-GPU); the NCCL form is dkv_decode(partial_out) +
 * all-gather + dkv_merge_partials.
 */
typedef struct dkv_exchange dkv_exchange;
int dkv_exchange_create(dkv_context* ctx, int rank, int world, int64_t max_rows, dkv_exchange** out);
int dkv_exchange_handle(dkv_exchange* ex, void* handle_out_64_bytes);
int dkv_exchange_connect(dkv_exchange* ex, int peer_rank, const void* handle_64_bytes);
/* Same-process form (one process driving several GPUs with peer access enabled, or several logical ranks on
 * one GPU): the peer's buffer address instead of an IPC handle. */
int dkv_exchange_base(dkv_exchange* ex, void** base_out);
int dkv_exchange_connect_ptr(dkv_exchange* ex, int peer_rank, void* peer_base);
int dkv_exchange_destroy(dkv_exchange* ex);
int dkv_decode_exchange(dkv_context* ctx, dkv_exchange* ex, const dkv_decode_args* args, void* out, float* lse,
                        void* stream);

/*
 * Same argument meaning as the reference's smpv2_fwd(X, Wk, Wv, Q, K_cpu, V_cpu, cos_sin,
 * softmax_scale, is_causal, seqlen_past, q_pos_start) -> O
 * (directkv/kernel/smpv2_extension.cu:574-637): projects the S_new new rows, rotates K at
 * positions seqlen_past.., stores them into K_cpu/V_cpu[:, seqlen_past:], and attends every new
 * row over past + new rows (causal offset seqlen_past).  Differences: the projection runs over
 * the full hidden size, and seqlen_past / S_new need not be multiples of 64.
 * X [B,S_new,H], Q/O [B,S_new,nh_q,128] device; K_cpu/V_cpu [B,S_total,nh_kv,128] pinned host
 * or device, S_total == seqlen_past + S_new.
 */
int dkv_smpv2_fwd(dkv_context* ctx, const void* X, const void* Wk, const void* Wv, const void* Q, void* K_cpu,
                  void* V_cpu, const float* cos_sin, int max_pos, int B, int S_new, int H, int nh_q, int nh_kv,
                  int S_total, float softmax_scale, int is_causal, int seqlen_past, int q_pos_start, void* O,
                  void* stream);

/*
 * Graph-safe form, replacing smpv2_fwd_graph (directkv/kernel/smpv2_extension.cu:436-569): the
 * layer must be registered; the number of past 64-token blocks is read from device memory
 * (n_past_blocks_dev, int32) when the work runs; req_pool_indices ([B] int32 device or NULL)
 * maps batch position to pool row (csrc/directKV_kernel.cuh:224-226).  Allocates nothing after
 * dkv_context_reserve.
 */
int dkv_smpv2_fwd_graph(dkv_context* ctx, int layer_id, const void* X_pad, const void* Q_pad, void* O_out,
                        const int32_t* n_past_blocks_dev, int B, int S_new, int nh_q, float softmax_scale,
                        int is_causal, const int32_t* req_pool_indices, void* stream);

/*
 * Extend / chunked prefill of registered pool rows: the kernel call of
 * DirectKVBackend.forward_extend (directkv/directkv_backend.py:681-697) without rebuilding
 * descriptors.  Request b uses pool row row_map[b] (or b); its S_new new rows are projected,
 * rotated at positions seqlen_past.., stored at [row, seqlen_past + i] and attend past + new
 * rows.  X [B,S_new,H], Q/O [B,S_new,nh_q,128] bf16 device.
 */
int dkv_extend(dkv_context* ctx, int layer_id, const void* X, const void* Q, void* O, int B, int S_new, int nh_q,
               float softmax_scale, int is_causal, int seqlen_past, int q_pos_start, const int32_t* row_map,
               void* stream);

/*
 * Attention of S_new rows that are ALREADY in the pool (stored by dkv_scatter_kv / set_kv_buffer) over
 * positions [0, seqlen_past + i] of their request, on the tensor-core extend kernel: the engine's form of
 * _sdpa_extend_manual (directkv/directkv_backend.py:861-891: gather req_to_token[req, :prefix + i + 1], triu mask
 * with diagonal prefix + 1).  page_table == NULL: contiguous rows (slot = row_map[b] * row_stride + position).
 * page_table [rows, pt_stride] int32 device: slot = page_table[row_map[b], position / page] * page + position % page
 * with the layer's page size (1 for SGLang's req_to_token); the request's rows are gathered once into a
 * contiguous staging tensor in HBM, which the kernel then reads once per 256 query rows.
 * Q/O [B, S_new, nh_q, 128] bf16 device.
 */
int dkv_extend_attend(dkv_context* ctx, int layer_id, const void* Q, void* O, int B, int S_new, int nh_q,
                      float softmax_scale, int is_causal, int seqlen_past, const int32_t* row_map,
                      const int32_t* page_table, int64_t pt_stride, void* stream);

/*
 * Extend of a RAGGED batch in one launch sequence: request b has s_new[b] new rows on past[b] stored rows and
 * uses pool row (or page-table row) rows[b]; the three arrays are HOST memory ([B] int32).  X [T, H] (or NULL:
 * the rows are in the pool already) and Q / O [T, nh_q, 128] hold the requests' rows one after the other,
 * T = sum of s_new.  The reference loops over the requests with one kernel call each
 * (directkv/directkv_backend.py:681-697); here the (request, query tile) pairs of the whole batch form one work
 * list, longest first, for one launch of the extend kernel.  Not capturable in a CUDA graph (host-side lengths).
 */
int dkv_extend_ragged(dkv_context* ctx, int layer_id, const void* X, const void* Q, void* O, int B,
                      const int32_t* s_new_host, const int32_t* past_host, const int32_t* rows_host, int nh_q,
                      float softmax_scale, int is_causal, const int32_t* page_table, int64_t pt_stride, void* stream);

/*
 * Stream-ordered store of new tokens into a token-indexed pool: replaces the blocking
 * device-to-host copy plus CPU scatter of DirectKVTokenToKVPool.set_kv_buffer
 * (directkv/directkv_pool.py:174-209).  Row i of cache_k / cache_v ([n_tokens, row_bytes],
 * device) is written to slot loc[i] of the pool ([n_slots, row_bytes], host-pinned or device)
 * by a kernel, with no host synchronisation.  loc is int32 or int64 in device memory.
 */
int dkv_scatter_kv(dkv_context* ctx, void* k_pool, void* v_pool, int64_t n_slots, int64_t k_row_bytes,
                   int64_t v_row_bytes, const void* loc, int loc_is_int64, const void* cache_k, const void* cache_v,
                   int64_t n_tokens, void* stream);

/*
 * Decode attention that allocates nothing.  It has no counterpart in the reference: it exists
 * for callers that may not allocate device memory when they call in - code running during
 * CUDA-graph capture, serving loops whose memory plan is frozen after start-up (all free HBM
 * already belongs to the KV-cache allocator), and host processes that forbid cudaMalloc /
 * cudaFree from plugins because those calls synchronise the device.  It needs no dkv_context:
 * its scratch is a fixed 4 MiB array inside the library (present on every GPU that loads the
 * library, for the life of the process).
 *
 * It computes what dkv_decode computes with new_mode == DKV_NEW_NONE over a paged pool: every
 * attended token is already in the pool; out[b] = softmax(q[b] K^T * scale) V per head.
 *
 * Limits and rules
 *  - sizes: batch <= 1983 and
 *      (SMs * W + batch * nh_kv * nsub) * G * 528 bytes <= 4 MiB - 8 KiB,
 *    with G = 4, 2 or 1 query heads handled together (the largest that divides nh_q / nh_kv),
 *    nsub = (nh_q / nh_kv) / G and W = 8 warps for G == 4, else 16.  On a 148-SM B200 that is,
 *    for example, 32 MHA heads up to batch 173, or Llama-3-8B's 32:8 GQA up to batch 99.  Larger
 *    sizes are rejected with DKV_ERR_UNSUPPORTED and a message that names both byte counts.
 *  - the first call on a device looks up the scratch array's device address and raises the
 *    kernels' shared-memory limit; make that call before any stream capture begins.
 *  - all calls share the one scratch array, which keeps the previous call's contents (the call
 *    clears the status word it needs at zero itself).  Calls that overlap on the GPU race:
 *    keep them on one stream or order them with events.
 *  - errors: the message is written to err_buf (when given); dkv_last_error() is not used.
 *  - the call runs on the current device (cudaGetDevice) and the given stream; q, out and a pool in device
 *    memory must belong to that device (a pool on another GPU is rejected), n_slots must be below 2^31.
 *  - a device-side failure (a bounded wait that ran out, a length that leads outside the page table) is
 *    reported by sync_and_check, or, without a synchronising call, through status_out.
 */
typedef struct {
    void*          k_pool;        /* [n_slots, nh_kv, 128] bf16; host-pinned or device */
    void*          v_pool;
    int64_t        n_slots;
    int            nh_kv;
    int            page_size;     /* power of two */
    int            batch;
    int            nh_q;
    const void*    q;             /* bf16 device, row b at q + b * q_stride, [nh_q, 128] */
    int64_t        q_stride;
    void*          out;           /* bf16 device, row b at out + b * out_stride */
    int64_t        out_stride;
    const int32_t* seq_lens;      /* [batch] int32 device: tokens attended, all in the pool */
    const int32_t* page_table;    /* [batch, pt_stride] int32 device */
    int            pt_stride;
    float          softmax_scale;
    float*         lse_out;       /* [batch, nh_q] or NULL */
    int            sync_and_check;/* non-zero: wait for the stream and report a device-side failure */
    char*          err_buf;       /* optional buffer for the error text */
    int            err_buf_len;
    unsigned int*  status_out;    /* optional device word of the caller's (current device): the kernels OR their
                                     DKV_STATUS_* bits into it instead of the library's own word, which the next
                                     call would clear - the way to notice a device-side failure of a call that was
                                     not made with sync_and_check.  The caller zeroes and reads it. */
} dkv_noalloc_args;

int dkv_decode_noalloc(const dkv_noalloc_args* args, void* stream);

/* Measurement aid, not part of the drop-in surface (no counterpart in the reference): a device-side copy
 * kernel reading `bytes` from src (host-mapped or device) into dst (device) with plain vector loads, to find
 * what reads issued by the SMs reach over the host link of a given machine. */
int dkv_stream_copy(dkv_context* ctx, void* dst, const void* src, int64_t bytes, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* DIRECTKV_B200_H */
