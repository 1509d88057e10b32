// C ABI of the engine (see include/directkv_b200.h): context, per-layer TMA descriptors,
// scratch management, argument checks and kernel launches.  Built with nvcc for sm_100a into
// libdirectkv_b200.so; depends only on the CUDA runtime (the one driver entry point it needs,
// cuTensorMapEncodeTiled, is looked up at run time so the library loads on a machine
// without a GPU driver).
#include "../../include/directkv_b200.h"

#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <algorithm>
#include <map>
#include <string>
#include <utility>
#include <vector>

#include "dkv_attn.cuh"
#include "dkv_attn_mma.cuh"
#include "dkv_proj_decode.cuh"
#include "dkv_proj_gemv.cuh"
#include "dkv_extend_pp.cuh"
#include "dkv_extend.cuh"
#include "dkv_proj.cuh"

namespace {

using namespace dkv;

thread_local std::string g_last_error;

int fail(int code, const char* fmt, ...) {
    char buf[1024];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof(buf), fmt, ap);
    va_end(ap);
    g_last_error = buf;
    return code;
}

#define DKV_CUDA(expr)                                                                              \
    do {                                                                                            \
        cudaError_t _e = (expr);                                                                    \
        if (_e != cudaSuccess)                                                                      \
            return fail(DKV_ERR_CUDA, "%s failed: %s (%s:%d)", #expr, cudaGetErrorString(_e), __FILE__, __LINE__); \
    } while (0)

#define DKV_REQUIRE(cond, ...)                           \
    do {                                                 \
        if (!(cond)) return fail(DKV_ERR_INVALID, __VA_ARGS__); \
    } while (0)

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (fn) return fn;
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) != cudaSuccess ||
        qres != cudaDriverEntryPointSuccess)
        return nullptr;
    fn = reinterpret_cast<EncodeTiledFn>(p);
    return fn;
}

// KV pool [n_slots, nh, 128] bf16 as a 3-D map (d, head, slot); one box = `rows` token rows of one head.
int encode_pool_map(CUtensorMap* m, void* base, int64_t n_slots, int nh, int rows) {
    EncodeTiledFn fn = get_encode_fn();
    if (!fn) return fail(DKV_ERR_CUDA, "cuTensorMapEncodeTiled entry point not available");
    cuuint64_t gdim[3] = {128, (cuuint64_t)nh, (cuuint64_t)n_slots};
    cuuint64_t gstr[2] = {256, (cuuint64_t)nh * 256};
    cuuint32_t box[3] = {128, 1, (cuuint32_t)rows};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, base, gdim, gstr, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(DKV_ERR_CUDA, "cuTensorMapEncodeTiled(pool) failed: %d", (int)r);
    return DKV_OK;
}

// Row-major [rows, cols] bf16 matrix as a 2-D map; box = 128 rows x 64 columns, 128-byte swizzle.
int encode_operand_map(CUtensorMap* m, const void* base, int64_t rows, int64_t cols, int box_rows = 128) {
    EncodeTiledFn fn = get_encode_fn();
    if (!fn) return fail(DKV_ERR_CUDA, "cuTensorMapEncodeTiled entry point not available");
    cuuint64_t gdim[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t gstr[1] = {(cuuint64_t)cols * 2};
    cuuint32_t box[2] = {64, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), gdim, gstr, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(DKV_ERR_CUDA, "cuTensorMapEncodeTiled(operand) failed: %d", (int)r);
    return DKV_OK;
}

// [rows, nh, 128] bf16 as a 3-D map (d, head, row); box = 64 columns x `box_heads` x `box_rows`, 128-byte swizzle:
// the operand tiles of the tensor-core extend kernel (K/V: one head, 128 rows; Q: G heads of 128/G tokens).
int encode_tile_map(CUtensorMap* m, const void* base, int64_t rows, int nh, int box_heads, int box_rows) {
    EncodeTiledFn fn = get_encode_fn();
    if (!fn) return fail(DKV_ERR_CUDA, "cuTensorMapEncodeTiled entry point not available");
    cuuint64_t gdim[3] = {128, (cuuint64_t)nh, (cuuint64_t)rows};
    cuuint64_t gstr[2] = {256, (cuuint64_t)nh * 256};
    cuuint32_t box[3] = {64, (cuuint32_t)box_heads, (cuuint32_t)box_rows};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), gdim, gstr, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(DKV_ERR_CUDA, "cuTensorMapEncodeTiled(tile) failed: %d", (int)r);
    return DKV_OK;
}

struct LayerState {
    dkv_layer_desc d{};
    void* k_dev = nullptr;  // device-visible address of the pool
    void* v_dev = nullptr;
    CUtensorMap tmK_page{}, tmV_page{};  // box rows = min(16, page_size)
    CUtensorMap tmK_16{}, tmV_16{};      // box rows = 16 (contiguous rows)
    CUtensorMap tmK_sw_page{}, tmV_sw_page{};  // 64 columns x rows_per_box, 128-byte swizzle (mma streaming kernel)
    CUtensorMap tmK_sw_16{}, tmV_sw_16{};
    CUtensorMap tmK_128{}, tmV_128{};    // 128 rows x 64 columns, 128-byte swizzle (tensor-core extend)
    CUtensorMap tmWk{}, tmWv{};
    int page_shift = 0;
    int rows_per_box = 16;
    bool has_weights = false;
    bool pool_on_host = false;
};

constexpr int kMaxCounters = 4096;

}  // namespace

// A device buffer that grows on demand.  Launches recorded by a stream capture keep the address they were given
// for as long as the graph lives, so a buffer that a capture has seen is never freed before the context is
// destroyed: when it has to grow, the old allocation is retired instead.
struct DevBuffer {
    uint8_t* ptr = nullptr;
    size_t bytes = 0;
    bool in_graph = false;              // a stream capture recorded launches that point into this allocation
};

struct dkv_context {
    int device = 0;
    int sm_count = 0;
    DevBuffer scratch;                  // per-call tables, partial records, new-token rows, split-K slices
    DevBuffer stage;                    // extend over a host or paged pool: the requests' rows gathered in HBM
    std::vector<void*> retired;         // outgrown allocations that a captured graph may still use
    unsigned int* status = nullptr;     // device status word
    unsigned int* counters = nullptr;   // split-K arrival counters, zero between launches
    std::map<int, LayerState> layers;
    cudaStream_t side = nullptr;        // projection overlaps the streamed attention here
    cudaEvent_t ev_fork = nullptr, ev_join = nullptr;
    int attn_variant = -1;              // -1: chosen per call from the head grouping
    int attn_ctas = 0;
    int attn_min_units = 5;          // HBM pools: a step with fewer (head-slot, tile) units per warp of the streaming grid than
                                     // this is split the short-step way (warp_split)
    int proj_split_k = 0;
    int wait_limit_ms = 2000;           // limit of the exchange consumer's wait for its peers
    int attn_self_scan = 1;             // batches of up to 32: no prep launch, the kernels scan the lengths themselves
    int proj_wide = 1;                  // 256-token projection tiles when there are more 128-token tiles than SMs
    int proj_gemv = 1;                  // one or two tokens into a device pool: matrix-vector kernel on the CUDA cores
    int proj_decode = -1;               // swapped-operand projection kernel: -1 when it can run under the streaming kernel; 0 never; 1 whenever T <= 512
    int attn_mma8 = 1;                  // tensor-core form with the query heads on the N side when <= 8 share a KV head (0: 16-row form)
    int attn_mma = -1;                  // -1: tensor-core inner product when 2..16 query heads share a KV head of an HBM pool; 0 never; 1 always
    int extend_pingpong = 1;            // two query tiles per CTA with specialised warps (0: one tile, four warps)
    int extend_rowwise = 0;             // 1: extend attends row by row with the decode kernels (reference path for tests)
    // Profiling: kernel launches issued, and CUDA-event pairs around the streaming kernel.
    long long launches = 0;
    int profile_attn = 0;
    std::vector<std::pair<cudaEvent_t, cudaEvent_t>> attn_events;
    size_t attn_events_used = 0;
    // Per-request metadata of a ragged extend: pinned host mirror, device copy, and the event of the last upload.
    int* ragged_host = nullptr;
    int* ragged_dev = nullptr;
    size_t ragged_ints = 0;
    cudaEvent_t ev_ragged = nullptr;
    bool ragged_pending = false;
};

// Peer-memory exchange of sequence-split partials (one per process group of <= 8 GPUs of a box).
struct dkv_exchange {
    dkv_context* ctx = nullptr;
    int rank = 0, world = 0;
    long long max_rows = 0;
    // cudaMalloc: records [2, world, max_rows, 132] fp32, then counters [2, kMaxExchangeRanks].  The leading 2 is
    // the parity of the step: consecutive steps use different halves, so a rank that runs one step ahead of a
    // peer (it cannot be further ahead, see dkv_decode_exchange) never stores over records the peer still reads.
    uint8_t* local = nullptr;
    size_t part_bytes = 0;
    size_t half_floats = 0;                                  // floats of one parity half of the record area
    float* part[dkv::kMaxExchangeRanks] = {nullptr};         // every rank's record area, as mapped into this process
    unsigned int* count[dkv::kMaxExchangeRanks] = {nullptr}; // every rank's arrival counters
    void* opened[dkv::kMaxExchangeRanks] = {nullptr};        // IPC mappings to close
    unsigned int expected[2][dkv::kMaxExchangeRanks] = {{0}}; // rows each rank has delivered so far, per parity (cumulative)
    unsigned long long steps = 0;                            // calls of dkv_decode_exchange so far
};

namespace {

// ---------------------------------------------------------------------------
// Small kernels that live with the host logic
// ---------------------------------------------------------------------------

// Extend: every new row becomes a virtual request that attends past + its causal prefix.
__global__ void extend_prep_kernel(int B, int S_new, int seqlen_past_host, const int* __restrict__ n_past_blocks_dev,
                                   int is_causal, const int* __restrict__ row_map, long long row_stride,
                                   int* __restrict__ vseq, int* __restrict__ vrow, int* __restrict__ tok_pos,
                                   int* __restrict__ tok_slot, int stage_stride, int* __restrict__ tok_stage_slot) {
    const int v = blockIdx.x * blockDim.x + threadIdx.x;
    if (v >= B * S_new) return;
    const int b = v / S_new, i = v - b * S_new;
    const int past = n_past_blocks_dev ? n_past_blocks_dev[0] * 64 : seqlen_past_host;
    const int row = row_map ? row_map[b] : b;
    vseq[v] = is_causal ? past + i + 1 : past + S_new;
    vrow[v] = row;
    tok_pos[v] = past + i;
    tok_slot[v] = static_cast<int>(static_cast<long long>(row) * row_stride + past + i);
    if (tok_stage_slot != nullptr) tok_stage_slot[v] = b * stage_stride + past + i;   // row of the staging copy [B, stage_stride]
}

// Largest b with prefix[b] <= v (prefix ascending, prefix[0] == 0).
__device__ __forceinline__ int find_request(const int* __restrict__ prefix, int n, long long v) {
    int lo = 0, hi = n - 1;
    while (lo < hi) {
        const int mid = (lo + hi + 1) >> 1;
        if (prefix[mid] <= v) lo = mid;
        else hi = mid - 1;
    }
    return lo;
}

// Ragged extend: position and pool slot of every new row of the packed batch.
// kv_off != nullptr: the new rows are projected into the staging copy (request b starts at row kv_off[b]) and
// tok_pool_slot receives the slot of the layer's own pool, for the write-back that follows.
__global__ void extend_prep_ragged_kernel(int B, int T, const int* __restrict__ q_row0, const int* __restrict__ past,
                                          const int* __restrict__ rows, long long row_stride, const int* __restrict__ kv_off,
                                          int* __restrict__ tok_pos, int* __restrict__ tok_slot,
                                          int* __restrict__ tok_pool_slot) {
    const int v = blockIdx.x * blockDim.x + threadIdx.x;
    if (v >= T) return;
    const int b = find_request(q_row0, B, v);
    const int i = v - q_row0[b];
    tok_pos[v] = past[b] + i;
    const int pool_slot = static_cast<int>(static_cast<long long>(rows[b]) * row_stride + past[b] + i);
    if (kv_off != nullptr) {
        tok_slot[v] = kv_off[b] + past[b] + i;
        tok_pool_slot[v] = pool_slot;
    } else {
        tok_slot[v] = pool_slot;
    }
}

// Write-back of freshly projected rows from the staging copy to the layer's (host) pool: one warp per row and
// tensor half, 16-byte stores; runs on the side stream while the attention reads the staging copy.
__global__ void __launch_bounds__(256) unstage_rows_kernel(uint4* __restrict__ k_pool, uint4* __restrict__ v_pool,
                                                           const uint4* __restrict__ k_stage, const uint4* __restrict__ v_stage,
                                                           const int* __restrict__ stage_slot, const int* __restrict__ pool_slot,
                                                           long long n_rows, int row_vec, long long n_slots,
                                                           unsigned int* status) {
    const long long total = n_rows * row_vec;
    const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
    for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
        const long long r = i / row_vec, c = i - r * row_vec;
        const long long dst = pool_slot[r];
        if (dst < 0 || dst >= n_slots) {
            if (c == 0) atomicOr(status, dkv::kStatusBadSlot);
            continue;
        }
        k_pool[dst * row_vec + c] = k_stage[static_cast<long long>(stage_slot[r]) * row_vec + c];
        v_pool[dst * row_vec + c] = v_stage[static_cast<long long>(stage_slot[r]) * row_vec + c];
    }
}

// Ragged extend over a host or paged pool: rows [0, past_b + s_new_b) of every request, one after the other, into
// a contiguous device staging tensor (request b starts at row kv_off[b]).
__global__ void __launch_bounds__(256) stage_rows_ragged_kernel(uint4* __restrict__ k_dst, uint4* __restrict__ v_dst,
                                                                const uint4* __restrict__ k_src,
                                                                const uint4* __restrict__ v_src, int B,
                                                                const int* __restrict__ kv_off,
                                                                const int* __restrict__ rows, long long row_stride,
                                                                int row_vec, const int* __restrict__ page_table,
                                                                long long pt_stride, int page_shift,
                                                                const int* __restrict__ past_only) {
    const long long total = static_cast<long long>(kv_off[B]) * row_vec;
    const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
    for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
        const long long srow = i / row_vec;
        const int b = find_request(kv_off, B, srow);
        const long long pos = srow - kv_off[b];
        if (past_only != nullptr && pos >= past_only[b]) continue;   // the new rows are projected straight into the copy
        const long long row = rows[b];
        long long slot;
        if (page_table != nullptr)
            slot = (static_cast<long long>(page_table[row * pt_stride + (pos >> page_shift)]) << page_shift) +
                   (pos & ((1ll << page_shift) - 1));
        else
            slot = row * row_stride + pos;
        const long long src = slot * row_vec + (i - srow * row_vec);
        k_dst[i] = __ldg(k_src + src);
        v_dst[i] = __ldg(v_src + src);
    }
}

// DKV_NEW_GIVEN: pack the caller's K/V rows into kv_new [B, nh, 2, 128] and store them to the pool.
__global__ void store_new_kv_kernel(const __nv_bfloat16* __restrict__ k_new, const __nv_bfloat16* __restrict__ v_new,
                                    int batch, int nh, const int* __restrict__ tok_slot, __nv_bfloat16* k_pool,
                                    __nv_bfloat16* v_pool, long long n_slots, __nv_bfloat16* __restrict__ kv_new,
                                    unsigned int* status) {
    const int lane = threadIdx.x & 31;
    const long long w = static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (w >= static_cast<long long>(batch) * nh) return;
    const int b = static_cast<int>(w / nh), h = static_cast<int>(w % nh);
    const __nv_bfloat16* src = (lane < 16 ? k_new : v_new) + (static_cast<long long>(b) * nh + h) * 128 + (lane & 15) * 8;
    const uint4 val = *reinterpret_cast<const uint4*>(src);
    *reinterpret_cast<uint4*>(kv_new + (static_cast<long long>(b) * nh + h) * 256 + lane * 8) = val;
    const long long slot = tok_slot[b];
    if (slot >= 0) {
        if (slot < n_slots) {
            __nv_bfloat16* dst = (lane < 16 ? k_pool : v_pool) + (slot * nh + h) * 128 + (lane & 15) * 8;
            *reinterpret_cast<uint4*>(dst) = val;
        } else if (lane == 0) {
            atomicOr(status, kStatusBadSlot);
        }
    }
}

// Optional Neox rotation of Q rows at positions q_pos_start + i (csrc/directKV_kernel.cuh:619-638).
__global__ void rope_q_kernel(const __nv_bfloat16* __restrict__ q, __nv_bfloat16* __restrict__ q_rot, int B, int S_new,
                              int nh_q, const float* __restrict__ cos_sin, int max_pos, int q_pos_start,
                              unsigned int* status) {
    const long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    const long long total = static_cast<long long>(B) * S_new * nh_q * 64;
    if (idx >= total) return;
    const int d = static_cast<int>(idx & 63);
    const long long rh = idx >> 6;  // (b, i, head)
    const int i = static_cast<int>((rh / nh_q) % S_new);
    const int pos = q_pos_start + i;
    const float lo = __bfloat162float(q[rh * 128 + d]), hi = __bfloat162float(q[rh * 128 + 64 + d]);
    float c = 1.f, s = 0.f;
    if (pos >= 0 && pos < max_pos) {
        c = cos_sin[static_cast<long long>(pos) * 128 + d];
        s = cos_sin[static_cast<long long>(pos) * 128 + 64 + d];
    } else {
        atomicOr(status, kStatusBadPosition);
    }
    q_rot[rh * 128 + d] = __float2bfloat16_rn(lo * c - hi * s);
    q_rot[rh * 128 + 64 + d] = __float2bfloat16_rn(hi * c + lo * s);
}

// Token-pool store: row i of src [n, row_bytes] goes to slot loc[i] of dst [n_slots, row_bytes].
// One CTA per token; 16-byte stores (row_bytes is a multiple of 16).
template <typename IndexT>
__global__ void __launch_bounds__(128) scatter_rows_kernel(uint4* __restrict__ dst, const uint4* __restrict__ src,
                                                           const IndexT* __restrict__ loc, long long n_slots,
                                                           int row_vec, unsigned int* status) {
    const long long i = blockIdx.x;
    const long long slot = static_cast<long long>(loc[i]);
    if (slot < 0 || slot >= n_slots) {
        if (threadIdx.x == 0) atomicOr(status, kStatusBadSlot);
        return;
    }
    for (int c = threadIdx.x; c < row_vec; c += blockDim.x) dst[slot * row_vec + c] = src[i * row_vec + c];
}

// Extend over a host pool: rows [0, s_total) of every request are brought into a device staging tensor
// [B, s_total, nh, 128] ONCE (16-byte read-only loads over the host link), so that the tensor-core kernel,
// which visits the keys once per 128-row query tile, re-reads them from HBM/L2 and not over PCIe.
__global__ void __launch_bounds__(256) stage_rows_kernel(uint4* __restrict__ k_dst, uint4* __restrict__ v_dst,
                                                         const uint4* __restrict__ k_src, const uint4* __restrict__ v_src,
                                                         const int* __restrict__ row_map, long long row_stride, int B,
                                                         int s_total, int row_vec /* nh * 16 */,
                                                         const int* __restrict__ page_table, long long pt_stride,
                                                         int page_shift, int past_only /* < 0: every row */) {
    const long long per_req = static_cast<long long>(s_total) * row_vec;
    const long long total = per_req * B;
    const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
    for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
        const int b = static_cast<int>(i / per_req);
        const long long r = i - b * per_req;
        const long long row = row_map ? row_map[b] : b;
        if (past_only >= 0 && r / row_vec >= past_only) continue;    // the new rows are projected straight into the copy
        long long src;
        if (page_table != nullptr) {
            // Paged pool: position -> slot through the request's row of the page table; the staged copy is contiguous.
            const long long pos = r / row_vec;
            const long long slot = (static_cast<long long>(page_table[row * pt_stride + (pos >> page_shift)]) << page_shift) +
                                   (pos & ((1ll << page_shift) - 1));
            src = slot * row_vec + (r - pos * row_vec);
        } else {
            src = row * row_stride * row_vec + r;
        }
        k_dst[i] = __ldg(k_src + src);
        v_dst[i] = __ldg(v_src + src);
    }
}

// Plain streaming copy (16-byte read-only loads), for measuring what SM-issued reads of
// host-mapped memory reach on this machine's host link.
__global__ void __launch_bounds__(256) stream_copy_kernel(uint4* __restrict__ dst, const uint4* __restrict__ src,
                                                          long long n16) {
    const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
    for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n16; i += stride)
        dst[i] = __ldg(src + i);
}

// ---------------------------------------------------------------------------
// Launch helpers
// ---------------------------------------------------------------------------
template <int G, int NW, int NST>
constexpr size_t attn_smem_bytes() {
    return attn_dyn_smem_bytes<NW, NST>();
}

template <int G, int NW, int NST>
cudaError_t attn_set_attr() {
    return cudaFuncSetAttribute(attn_partial_kernel<G, NW, NST>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                static_cast<int>(attn_smem_bytes<G, NW, NST>()));
}

template <int G, int NW, int NST>
cudaError_t attn_launch(int ctas, const CUtensorMap& tmK, const CUtensorMap& tmV, const AttnParams& p,
                        cudaStream_t st) {
    attn_partial_kernel<G, NW, NST><<<ctas, NW * 32, attn_smem_bytes<G, NW, NST>(), st>>>(tmK, tmV, p);
    return cudaGetLastError();
}

// Warps per CTA of the selectable variants of the streaming kernel (stages: 3, 2, 1).
constexpr int kVarWarps[3] = {8, 12, 16};

template <int G>
cudaError_t attn_dispatch(int variant, int ctas, const CUtensorMap& tmK, const CUtensorMap& tmV, const AttnParams& p,
                          cudaStream_t st) {
    switch (variant) {
        case 1: return attn_launch<G, 12, 2>(ctas, tmK, tmV, p, st);
        case 2: if (G <= 2) return attn_launch<(G <= 2 ? G : 1), 16, 1>(ctas, tmK, tmV, p, st);
                return attn_launch<G, 12, 2>(ctas, tmK, tmV, p, st);
        default: return attn_launch<G, 8, 3>(ctas, tmK, tmV, p, st);
    }
}

template <int NW, int NST>
cudaError_t attn_mma_launch(int ctas, const CUtensorMap& tmK, const CUtensorMap& tmV, const AttnParams& p, cudaStream_t st) {
    attn_partial_mma_kernel<NW, NST><<<ctas, NW * 32, attn_smem_bytes<1, NW, NST>(), st>>>(tmK, tmV, p);
    return cudaGetLastError();
}

cudaError_t attn_mma_dispatch(int variant, int ctas, const CUtensorMap& tmK, const CUtensorMap& tmV, const AttnParams& p,
                              cudaStream_t st) {
    switch (variant) {
        case 0: return attn_mma_launch<8, 3>(ctas, tmK, tmV, p, st);
        case 1: return attn_mma_launch<12, 2>(ctas, tmK, tmV, p, st);
        default: return attn_mma_launch<16, 1>(ctas, tmK, tmV, p, st);
    }
}

template <int NW, int NST>
cudaError_t attn_mma8_launch(int ctas, const CUtensorMap& tmK, const CUtensorMap& tmV, const AttnParams& p, cudaStream_t st) {
    attn_partial_mma8_kernel<NW, NST><<<ctas, NW * 32, attn_smem_bytes<1, NW, NST>(), st>>>(tmK, tmV, p);
    return cudaGetLastError();
}

cudaError_t attn_mma8_dispatch(int variant, int ctas, const CUtensorMap& tmK, const CUtensorMap& tmV, const AttnParams& p,
                               cudaStream_t st) {
    switch (variant) {
        case 0: return attn_mma8_launch<8, 3>(ctas, tmK, tmV, p, st);
        case 1: return attn_mma8_launch<12, 2>(ctas, tmK, tmV, p, st);
        default: return attn_mma8_launch<16, 1>(ctas, tmK, tmV, p, st);
    }
}

// Kernels that are meant to share an SM ask for the largest shared-memory carve-out, so that whichever of them
// arrives first does not leave the SM configured too small for the other.
template <typename K>
cudaError_t prefer_max_shared(K kernel) {
    return cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
}

template <int T>
cudaError_t set_gemv_attributes() {
    cudaError_t e = cudaFuncSetAttribute(proj_rope_gemv_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, kGvSmemBudget);
    return e != cudaSuccess ? e : prefer_max_shared(proj_rope_gemv_kernel<T>);
}

template <int NW, int NST>
cudaError_t attn_mma8_set_attr() {
    cudaError_t e = cudaFuncSetAttribute(attn_partial_mma8_kernel<NW, NST>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         static_cast<int>(attn_smem_bytes<1, NW, NST>()));
    return e != cudaSuccess ? e : prefer_max_shared(attn_partial_mma8_kernel<NW, NST>);
}

template <int NW, int NST>
cudaError_t attn_mma_set_attr() {
    return cudaFuncSetAttribute(attn_partial_mma_kernel<NW, NST>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                static_cast<int>(attn_smem_bytes<1, NW, NST>()));
}

constexpr int kProjStages = 4;       // 48 KB stages (128 tokens per CTA)
constexpr int kProjStagesWide = 3;   // 64 KB stages (256 tokens per CTA)
static_assert(kProjStagesWide * (2 * kProjABytes + kProjBBytes) == kProjStages * kProjStage, "both forms use the same ring size");
// stages | control (barriers, TMEM holder) | alignment slack; the epilogue re-uses the stage area for
// the split-K sum tile (128 x 260 floats) followed by the 64 KB bf16 output staging tile.
constexpr size_t kProjSmem = static_cast<size_t>(kProjStages) * kProjStage + 4096 + 1024 + 1024;

size_t align256(size_t x) { return (x + 255) & ~static_cast<size_t>(255); }

struct ScratchPlan {
    size_t cum, tok_pos, tok_slot, vseq, vrow, partials, kv_new, splitk, q_rot, total;   // offsets into ctx->scratch
    size_t stage_k, stage_v, stage_total;                                                // offsets into ctx->stage
};

// The tensor-core form reads 128-byte row segments (two 64-column swizzled boxes per row); over PCIe those make
// half-size read requests and cost 20 % of the link (40 against 51 GB/s), and the link, not the instruction
// issue rate, bounds a host-resident pool: automatic choice only for pools in HBM.
bool use_mma(const dkv_context* ctx, int g_total, bool pool_on_host) {
    return ctx->attn_mma == 1 || (ctx->attn_mma < 0 && g_total >= 2 && !pool_on_host);
}

// Query heads that share one pass over a KV head: the mma kernel takes up to 16 rows (the largest divisor of
// g_total that fits), the CUDA-core kernel 4, 2 or 1.
int choose_g(const dkv_context* ctx, int g_total, bool pool_on_host) {
    if (use_mma(ctx, g_total, pool_on_host)) {
        int g = g_total < 16 ? g_total : 16;
        while (g_total % g != 0) --g;
        return g;
    }
    return (g_total % 4 == 0) ? 4 : (g_total % 2 == 0) ? 2 : 1;
}

// Variant actually launched for a head grouping (measured on B200, KV in HBM): G == 1: 16 warps x 1 stage
// (6.5 TB/s); G == 2: 12 warps x 2 stages (6.1 TB/s); G == 4 needs 218 registers per thread and runs 8 warps
// x 3 stages (4.3 TB/s).
int effective_variant(const dkv_context* ctx, int G) {
    int v = ctx->attn_variant;
    if (v < 0) v = (G == 1) ? 2 : (G == 2) ? 1 : 0;
    if (v == 2 && G > 2) v = 1;
    return v;
}

int variant_warps(const dkv_context* ctx, int G) { return kVarWarps[effective_variant(ctx, G)]; }

int attn_cta_count(const dkv_context* ctx) { return ctx->attn_ctas > 0 ? ctx->attn_ctas : ctx->sm_count; }

void proj_split(const dkv_context* ctx, int T, int nh_kv, int H, int* split_k, int* cps) {
    const int tiles = ((T + kProjBM - 1) / kProjBM) * nh_kv;
    const int nchunks = H / kProjBK;
    int s = ctx->proj_split_k > 0 ? ctx->proj_split_k : ctx->sm_count / (tiles > 0 ? tiles : 1);
    if (s < 1) s = 1;
    if (s > nchunks) s = nchunks;
    if (tiles > kMaxCounters) s = 1;
    const int c = (nchunks + s - 1) / s;
    *cps = c;
    *split_k = (nchunks + c - 1) / c;  // no empty slice
}

// Split of the hidden dimension for the decode-batch projection: one CTA per (KV head, slice), about one
// CTA per SM, at least four 64-column chunks per slice.
void proj_decode_split(const dkv_context* ctx, int T, int nh_kv, int H, int* split_k, int* cps) {
    const int nchunks = H / kProjBK;
    const int units = nh_kv * ((T + kPdMaxTokens - 1) / kPdMaxTokens);       // (KV head, 128-token chunk) pairs
    int s = ctx->proj_split_k > 0 ? ctx->proj_split_k : ctx->sm_count / (units > 0 ? units : 1);
    if (ctx->proj_split_k <= 0 && s > nchunks / 4) s = nchunks / 4;
    if (s < 1) s = 1;
    if (s > nchunks) s = nchunks;
    if (units > kMaxCounters) s = 1;
    const int c = (nchunks + s - 1) / s;
    *cps = c;
    *split_k = (nchunks + c - 1) / c;
}

ScratchPlan plan_scratch(const dkv_context* ctx, int64_t rows, int nh_q, int nh_kv, int hidden, bool with_proj,
                         bool with_qrot, size_t stage_bytes = 0) {
    ScratchPlan s{};
    const int g_total = nh_q / nh_kv;
    const size_t total_warps = static_cast<size_t>(attn_cta_count(ctx)) * 16;  // upper bound over variants
    // Partial records of whichever form of the streaming kernel runs (the choice depends on where the pool lives).
    size_t partial_floats = 0;
    for (int on_host = 0; on_host < 2; ++on_host) {
        const int G = choose_g(ctx, g_total, on_host != 0);
        const int nsub = g_total / G;
        const size_t f = (total_warps + static_cast<size_t>(rows) * nh_kv * nsub) * G * kPartialStride;
        partial_floats = f > partial_floats ? f : partial_floats;
    }
    size_t off = 0;
    s.cum = off;      off += align256((rows + 1) * 4);
    s.tok_pos = off;  off += align256(rows * 4);
    s.tok_slot = off; off += align256(rows * 4);
    s.vseq = off;     off += align256(rows * 4);
    s.vrow = off;     off += align256(rows * 4);
    s.partials = off; off += align256(partial_floats * 4);
    s.kv_new = off;   off += align256(static_cast<size_t>(rows) * nh_kv * 256 * 2);
    s.splitk = off;
    if (with_proj && hidden > 0) {
        int split_k, cps;
        proj_split(ctx, static_cast<int>(rows), nh_kv, hidden, &split_k, &cps);
        size_t bytes = 0;
        if (split_k > 1) {
            const size_t tiles = static_cast<size_t>((rows + kProjBM - 1) / kProjBM) * nh_kv;
            bytes = static_cast<size_t>(split_k) * tiles * kProjBM * kProjBN * 4;
        }
        // The decode-batch kernel (up to 128 rows) splits differently; a plan made for many rows also covers
        // a later call with few.
        // Worst case over the batches a later call may bring: one token chunk with the deepest split, or all chunks.
        for (int64_t t : {static_cast<int64_t>(rows < kPdMaxTokens ? rows : kPdMaxTokens),
                          static_cast<int64_t>(rows < kPdMaxBatch ? rows : kPdMaxBatch)}) {
            proj_decode_split(ctx, static_cast<int>(t), nh_kv, hidden, &split_k, &cps);
            if (split_k > 1) {
                const size_t box_rows = t > kPdMaxTokens ? kPdMaxTokens : pd_padded_tokens(static_cast<int>(t));
                const size_t n_chunks = (t + kPdMaxTokens - 1) / kPdMaxTokens;
                const size_t dec = static_cast<size_t>(split_k) * nh_kv * n_chunks * 2 * box_rows * kProjHead * 4;
                bytes = bytes > dec ? bytes : dec;
            }
        }
        off += align256(bytes);
    }
    s.q_rot = off;
    if (with_qrot) off += align256(static_cast<size_t>(rows) * nh_q * 128 * 2);
    s.total = off;
    s.stage_k = 0;
    s.stage_v = (stage_bytes + 1023) & ~static_cast<size_t>(1023);      // TMA bases: keep both halves 1 KB aligned
    s.stage_total = stage_bytes ? 2 * s.stage_v : 0;
    return s;
}

bool stream_is_capturing(cudaStream_t st) {
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(st, &cap) != cudaSuccess) {
        (void)cudaGetLastError();       // e.g. the legacy stream while another stream captures: not our capture
        return false;
    }
    return cap != cudaStreamCaptureStatusNone;
}

// Makes `b` hold at least `bytes`.  `capturing`: the calling entry point is being recorded into a CUDA graph.
// Growth never happens under capture (the caller must have reserved), and an allocation that any capture has
// seen is retired, not freed, so a later replay of that graph still finds its memory.
int ensure_buffer(dkv_context* ctx, DevBuffer* b, size_t bytes, bool capturing, const char* what) {
    if (bytes > b->bytes) {
        if (capturing)
            return fail(DKV_ERR_UNSUPPORTED,
                        "%s of %zu bytes needed during stream capture but %zu are reserved: size it before capturing "
                        "(dkv_context_reserve, or one eager call of the same shape)", what, bytes, b->bytes);
        uint8_t* p = nullptr;
        const size_t want = bytes + (bytes >> 2);
        DKV_CUDA(cudaMalloc(&p, want));
        if (b->ptr != nullptr) {
            if (b->in_graph) {
                ctx->retired.push_back(b->ptr);
            } else {
                DKV_CUDA(cudaDeviceSynchronize());      // launches in flight may still use the old allocation
                DKV_CUDA(cudaFree(b->ptr));
            }
        }
        b->ptr = p;
        b->bytes = want;
        b->in_graph = false;
    }
    if (capturing) b->in_graph = true;
    return DKV_OK;
}

int ensure_scratch(dkv_context* ctx, const ScratchPlan& sp, cudaStream_t st) {
    const bool capturing = stream_is_capturing(st);
    int rc = ensure_buffer(ctx, &ctx->scratch, sp.total, capturing, "scratch");
    if (rc != DKV_OK || sp.stage_total == 0) return rc;
    return ensure_buffer(ctx, &ctx->stage, sp.stage_total, capturing, "staging memory");
}

int device_pointer_of(void* p, void** out, const char* what) {
    cudaPointerAttributes attr;
    DKV_CUDA(cudaPointerGetAttributes(&attr, p));
    if (attr.type == cudaMemoryTypeDevice || attr.type == cudaMemoryTypeManaged) {
        *out = p;
        return DKV_OK;
    }
    if (attr.type == cudaMemoryTypeHost && attr.devicePointer != nullptr) {
        *out = attr.devicePointer;
        return DKV_OK;
    }
    return fail(DKV_ERR_INVALID, "%s must be pinned (page-locked) host memory or device memory", what);
}

int build_layer(LayerState* L, const dkv_layer_desc* d) {
    DKV_REQUIRE(d->k_pool && d->v_pool, "k_pool / v_pool must not be NULL");
    DKV_REQUIRE(d->n_slots > 0 && d->nh_kv > 0, "n_slots and nh_kv must be positive");
    // Slot numbers travel as 32-bit TMA coordinates and int32 page-table entries.
    DKV_REQUIRE(d->n_slots <= static_cast<int64_t>(INT32_MAX), "n_slots (%lld) exceeds the 2^31 - 1 slots a pool can address",
                (long long)d->n_slots);
    DKV_REQUIRE(d->page_size >= 1 && (d->page_size & (d->page_size - 1)) == 0, "page_size (%d) must be a power of two",
                d->page_size);
    DKV_REQUIRE((reinterpret_cast<uintptr_t>(d->k_pool) & 15) == 0 && (reinterpret_cast<uintptr_t>(d->v_pool) & 15) == 0,
                "KV pool base addresses must be 16-byte aligned");
    L->d = *d;
    int rc;
    {
        cudaPointerAttributes attr;
        DKV_CUDA(cudaPointerGetAttributes(&attr, d->k_pool));
        L->pool_on_host = (attr.type == cudaMemoryTypeHost);
    }
    if ((rc = device_pointer_of(d->k_pool, &L->k_dev, "k_pool")) != DKV_OK) return rc;
    if ((rc = device_pointer_of(d->v_pool, &L->v_dev, "v_pool")) != DKV_OK) return rc;
    L->page_shift = 0;
    while ((1 << L->page_shift) < d->page_size) ++L->page_shift;
    L->rows_per_box = d->page_size < kTileTokens ? d->page_size : kTileTokens;
    if ((rc = encode_pool_map(&L->tmK_page, L->k_dev, d->n_slots, d->nh_kv, L->rows_per_box)) != DKV_OK) return rc;
    if ((rc = encode_pool_map(&L->tmV_page, L->v_dev, d->n_slots, d->nh_kv, L->rows_per_box)) != DKV_OK) return rc;
    if ((rc = encode_pool_map(&L->tmK_16, L->k_dev, d->n_slots, d->nh_kv, kTileTokens)) != DKV_OK) return rc;
    if ((rc = encode_pool_map(&L->tmV_16, L->v_dev, d->n_slots, d->nh_kv, kTileTokens)) != DKV_OK) return rc;
    if ((rc = encode_tile_map(&L->tmK_sw_page, L->k_dev, d->n_slots, d->nh_kv, 1, L->rows_per_box)) != DKV_OK) return rc;
    if ((rc = encode_tile_map(&L->tmV_sw_page, L->v_dev, d->n_slots, d->nh_kv, 1, L->rows_per_box)) != DKV_OK) return rc;
    if ((rc = encode_tile_map(&L->tmK_sw_16, L->k_dev, d->n_slots, d->nh_kv, 1, kTileTokens)) != DKV_OK) return rc;
    if ((rc = encode_tile_map(&L->tmV_sw_16, L->v_dev, d->n_slots, d->nh_kv, 1, kTileTokens)) != DKV_OK) return rc;
    if ((rc = encode_tile_map(&L->tmK_128, L->k_dev, d->n_slots, d->nh_kv, 1, kExtTile)) != DKV_OK) return rc;
    if ((rc = encode_tile_map(&L->tmV_128, L->v_dev, d->n_slots, d->nh_kv, 1, kExtTile)) != DKV_OK) return rc;
    L->has_weights = (d->wk != nullptr && d->wv != nullptr);
    if (L->has_weights) {
        DKV_REQUIRE(d->hidden > 0 && d->hidden % kProjBK == 0, "hidden (%d) must be a positive multiple of 64", d->hidden);
        if ((rc = encode_operand_map(&L->tmWk, d->wk, static_cast<int64_t>(d->nh_kv) * 128, d->hidden)) != DKV_OK) return rc;
        if ((rc = encode_operand_map(&L->tmWv, d->wv, static_cast<int64_t>(d->nh_kv) * 128, d->hidden)) != DKV_OK) return rc;
    }
    if (d->cos_sin) DKV_REQUIRE(d->max_pos > 0, "max_pos must be positive when cos_sin is given");
    return DKV_OK;
}

// Projection of T rows of X with RoPE and write-back (tcgen05 kernel).
int launch_projection(dkv_context* ctx, const LayerState& L, const void* x, int T, const int* tok_pos,
                      const int* tok_slot, bool store_pool, __nv_bfloat16* kv_new, float* splitk, cudaStream_t st,
                      bool beside_streaming = false, void* k_dst = nullptr, void* v_dst = nullptr, long long n_slots_dst = 0,
                      const DecodePlace* place = nullptr) {
    // The swapped-operand kernel pays off where it runs UNDER the streaming kernel (the 16-warp CUDA-core form
    // leaves it registers and shared memory); alone, the 128-token-tile kernel with its deeper ring is faster.
    const bool small = T <= kPdMaxBatch && (ctx->proj_decode == 1 || (ctx->proj_decode < 0 && beside_streaming));
    // One or two tokens into a pool in device memory: a matrix-vector stream on the CUDA cores (two-byte stores
    // per dimension pair are fine for HBM, not for rows behind the host link).
    const bool tiny = ctx->proj_gemv != 0 && gv_supports(T, L.d.hidden) && k_dst == nullptr && !(store_pool && L.pool_on_host);
    ProjParams pp{};
    pp.T = T;
    pp.H = L.d.hidden;
    pp.nh_kv = L.d.nh_kv;
    if (small) proj_decode_split(ctx, T, L.d.nh_kv, L.d.hidden, &pp.split_k, &pp.chunks_per_split);
    else proj_split(ctx, T, L.d.nh_kv, L.d.hidden, &pp.split_k, &pp.chunks_per_split);
    // More 128-token tiles than SMs (prefill sizes): 256 tokens per CTA, so the weights cross L2 once per 256.
    const int tiles128 = (T + kProjBM - 1) / kProjBM;
    const bool wide = !small && pp.split_k == 1 && ctx->proj_wide != 0 &&
                      static_cast<long long>(tiles128) * L.d.nh_kv > ctx->sm_count;
    CUtensorMap tmX;
    const int pd_box_rows = T > kPdMaxTokens ? kPdMaxTokens : pd_padded_tokens(T);
    int rc = encode_operand_map(&tmX, x, T, L.d.hidden, small ? pd_box_rows : wide ? 256 : 128);
    if (rc != DKV_OK) return rc;
    pp.tok_pos = tok_pos;
    pp.tok_slot = tok_slot;
    if (place != nullptr) pp.place = *place;
    pp.cos_sin = L.d.cos_sin;
    pp.max_pos = L.d.max_pos;
    // The rows go to the layer's pool, or (k_dst given) to a staging copy of it whose slots tok_slot addresses.
    pp.k_pool = store_pool ? static_cast<__nv_bfloat16*>(k_dst ? k_dst : L.k_dev) : nullptr;
    pp.v_pool = store_pool ? static_cast<__nv_bfloat16*>(k_dst ? v_dst : L.v_dev) : nullptr;
    pp.n_slots = k_dst ? n_slots_dst : L.d.n_slots;
    pp.kv_new = kv_new;
    pp.splitk_scratch = splitk;
    pp.tile_counters = ctx->counters;
    pp.status = ctx->status;
    if (tiny) {
        const int ctas = (L.d.nh_kv * 128 + kGvWarps - 1) / kGvWarps;      // a warp per row pair at most
        const int grid = ctas < ctx->sm_count ? ctas : ctx->sm_count;
        const size_t smem = gv_smem_bytes(T, L.d.hidden);
        const __nv_bfloat16* xb = static_cast<const __nv_bfloat16*>(x);
        const __nv_bfloat16* wkb = static_cast<const __nv_bfloat16*>(L.d.wk);
        const __nv_bfloat16* wvb = static_cast<const __nv_bfloat16*>(L.d.wv);
        if (T == 1) proj_rope_gemv_kernel<1><<<grid, 128, smem, st>>>(xb, wkb, wvb, pp);
        else proj_rope_gemv_kernel<2><<<grid, 128, smem, st>>>(xb, wkb, wvb, pp);
    } else if (small) {
        dim3 grid(L.d.nh_kv, pp.split_k, (T + kPdMaxTokens - 1) / kPdMaxTokens);
        proj_rope_decode_kernel<<<grid, 128, pd_smem_bytes(pd_box_rows), st>>>(tmX, L.tmWk, L.tmWv, pp);
    } else if (wide) {
        dim3 grid(L.d.nh_kv, (tiles128 + 1) / 2, 1);
        proj_rope_kernel<kProjStagesWide, 2><<<grid, 128, kProjSmem, st>>>(tmX, L.tmWk, L.tmWv, pp);
    } else {
        dim3 grid(L.d.nh_kv, tiles128, pp.split_k);
        proj_rope_kernel<kProjStages, 1><<<grid, 128, kProjSmem, st>>>(tmX, L.tmWk, L.tmWv, pp);
    }
    DKV_CUDA(cudaGetLastError());
    ctx->launches += 1;
    return DKV_OK;
}

int launch_attention(dkv_context* ctx, const LayerState& L, AttnParams& ap, bool paged, const MergeParams& mp_in,
                     cudaStream_t st, cudaEvent_t join_before_merge = nullptr) {
    const int G = choose_g(ctx, ap.g_total, L.pool_on_host);
    const bool mma = use_mma(ctx, ap.g_total, L.pool_on_host);
    ap.nsub = ap.g_total / G;
    const int ctas = attn_cta_count(ctx);
    const int mma_variant = ctx->attn_variant < 0 ? 2 : ctx->attn_variant;
    ap.total_warps = ctas * (mma ? kVarWarps[mma_variant] : variant_warps(ctx, G));
    // Rows in host memory want every warp's loads in flight; rows in HBM want few partial records on short steps.
    ap.min_units = (L.pool_on_host || ctx->attn_min_units < 1) ? 1 : ctx->attn_min_units;
    const CUtensorMap& tmK = mma ? (paged ? L.tmK_sw_page : L.tmK_sw_16) : (paged ? L.tmK_page : L.tmK_16);
    const CUtensorMap& tmV = mma ? (paged ? L.tmV_sw_page : L.tmV_sw_16) : (paged ? L.tmV_page : L.tmV_16);
    cudaError_t e;
    std::pair<cudaEvent_t, cudaEvent_t>* ev = nullptr;
    if (ctx->profile_attn) {
        if (ctx->attn_events_used == ctx->attn_events.size() && ctx->attn_events.size() < 8192) {
            cudaEvent_t a, b;
            DKV_CUDA(cudaEventCreate(&a));
            DKV_CUDA(cudaEventCreate(&b));
            ctx->attn_events.emplace_back(a, b);
        }
        if (ctx->attn_events_used < ctx->attn_events.size()) ev = &ctx->attn_events[ctx->attn_events_used++];
    }
    if (ev) DKV_CUDA(cudaEventRecord(ev->first, st));
    if (mma && G <= 8 && ctx->attn_mma8 != 0) e = attn_mma8_dispatch(mma_variant, ctas, tmK, tmV, ap, st);
    else if (mma) e = attn_mma_dispatch(mma_variant, ctas, tmK, tmV, ap, st);
    else if (G == 4) e = attn_dispatch<4>(effective_variant(ctx, 4), ctas, tmK, tmV, ap, st);
    else if (G == 2) e = attn_dispatch<2>(effective_variant(ctx, 2), ctas, tmK, tmV, ap, st);
    else e = attn_dispatch<1>(effective_variant(ctx, 1), ctas, tmK, tmV, ap, st);
    DKV_CUDA(e);
    if (ev) DKV_CUDA(cudaEventRecord(ev->second, st));
    ctx->launches += 2;  // streaming kernel + merge
    if (join_before_merge) DKV_CUDA(cudaStreamWaitEvent(st, join_before_merge, 0));
    MergeParams mp = mp_in;
    mp.a = ap;
    mp.G = G;
    // Records per row are about (warps of the streaming grid) / (request x head-slot segments) + 2: with few
    // segments eight warps share a row.
    const long long rows = static_cast<long long>(ap.batch) * ap.nh_q;
    const long long segments = static_cast<long long>(ap.batch) * ap.nh_kv * ap.nsub;
    // A row can have at most (tiles of the longest request the addressing allows) / (tiles per warp) + 2 records; the
    // 32-warp form pays only when there can be more than 64.
    const long long max_tokens = paged ? static_cast<long long>(ap.pt_stride) * ap.page_size : ap.row_stride;
    const long long max_records = max_tokens / kTileTokens / ap.min_units + 2;
    if (segments * 64 < ap.total_warps && max_records > 64)
        attn_merge_kernel<32><<<static_cast<int>(rows), merge_threads(32), 0, st>>>(mp);
    else if (segments * 8 < ap.total_warps) attn_merge_kernel<8><<<static_cast<int>(rows), kMergeThreads, 0, st>>>(mp);
    else attn_merge_kernel<1><<<static_cast<int>((rows + 7) / 8), kMergeThreads, 0, st>>>(mp);
    DKV_CUDA(cudaGetLastError());
    return DKV_OK;
}

}  // namespace

// ===========================================================================
// Exported functions
// ===========================================================================
extern "C" {

int dkv_version(void) { return 100; }

const char* dkv_last_error(void) { return g_last_error.c_str(); }

int dkv_context_create(int device, dkv_context** out) {
    DKV_REQUIRE(out != nullptr, "out must not be NULL");
    int ndev = 0;
    DKV_CUDA(cudaGetDeviceCount(&ndev));
    DKV_REQUIRE(device >= 0 && device < ndev, "device %d out of range (%d devices)", device, ndev);
    DKV_CUDA(cudaSetDevice(device));
    cudaDeviceProp prop;
    DKV_CUDA(cudaGetDeviceProperties(&prop, device));
    if (prop.major != 10)
        return fail(DKV_ERR_UNSUPPORTED, "device %d is sm_%d%d; this library is built for sm_100a only", device,
                    prop.major, prop.minor);
    dkv_context* ctx = new dkv_context();
    ctx->device = device;
    ctx->sm_count = prop.multiProcessorCount;
    cudaError_t e = cudaMalloc(&ctx->status, sizeof(unsigned int));
    if (e == cudaSuccess) e = cudaMemset(ctx->status, 0, sizeof(unsigned int));
    if (e == cudaSuccess) e = cudaMalloc(&ctx->counters, kMaxCounters * sizeof(unsigned int));
    if (e == cudaSuccess) e = cudaMemset(ctx->counters, 0, kMaxCounters * sizeof(unsigned int));
    if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&ctx->side, cudaStreamNonBlocking);
    if (e == cudaSuccess) e = cudaEventCreateWithFlags(&ctx->ev_fork, cudaEventDisableTiming);
    if (e == cudaSuccess) e = cudaEventCreateWithFlags(&ctx->ev_join, cudaEventDisableTiming);
    if (e == cudaSuccess) e = attn_set_attr<1, 8, 3>();
    if (e == cudaSuccess) e = attn_set_attr<2, 8, 3>();
    if (e == cudaSuccess) e = attn_set_attr<4, 8, 3>();
    if (e == cudaSuccess) e = attn_set_attr<1, 12, 2>();
    if (e == cudaSuccess) e = attn_set_attr<2, 12, 2>();
    if (e == cudaSuccess) e = attn_set_attr<4, 12, 2>();
    if (e == cudaSuccess) e = attn_set_attr<1, 16, 1>();
    if (e == cudaSuccess) e = attn_set_attr<2, 16, 1>();
    if (e == cudaSuccess) e = attn_mma_set_attr<8, 3>();
    if (e == cudaSuccess) e = attn_mma_set_attr<12, 2>();
    if (e == cudaSuccess) e = attn_mma_set_attr<16, 1>();
    if (e == cudaSuccess) e = attn_mma8_set_attr<8, 3>();
    if (e == cudaSuccess) e = attn_mma8_set_attr<12, 2>();
    if (e == cudaSuccess) e = attn_mma8_set_attr<16, 1>();
    if (e == cudaSuccess)
        e = cudaFuncSetAttribute(extend_attn_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kExtSmem + 1024);
    if (e == cudaSuccess)
        e = cudaFuncSetAttribute(extend_attn_pp_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kPpSmem);
    if (e == cudaSuccess)
        e = cudaFuncSetAttribute(proj_rope_kernel<kProjStages, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 static_cast<int>(kProjSmem));
    if (e == cudaSuccess)
        e = cudaFuncSetAttribute(proj_rope_kernel<kProjStagesWide, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 static_cast<int>(kProjSmem));
    if (e == cudaSuccess)
        e = cudaFuncSetAttribute(proj_rope_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 static_cast<int>(pd_smem_bytes(kPdMaxTokens)));
    if (e == cudaSuccess) e = prefer_max_shared(proj_rope_decode_kernel);
    if (e == cudaSuccess) e = set_gemv_attributes<1>();
    if (e == cudaSuccess) e = set_gemv_attributes<2>();
    if (e == cudaSuccess) e = prefer_max_shared(attn_partial_kernel<1, 16, 1>);
    if (e != cudaSuccess) {
        delete ctx;
        return fail(DKV_ERR_CUDA, "context set-up failed: %s", cudaGetErrorString(e));
    }
    *out = ctx;
    return DKV_OK;
}

int dkv_context_destroy(dkv_context* ctx) {
    if (!ctx) return DKV_OK;
    cudaSetDevice(ctx->device);
    cudaDeviceSynchronize();
    for (auto& ev : ctx->attn_events) {
        cudaEventDestroy(ev.first);
        cudaEventDestroy(ev.second);
    }
    if (ctx->side) cudaStreamDestroy(ctx->side);
    if (ctx->ev_fork) cudaEventDestroy(ctx->ev_fork);
    if (ctx->ev_join) cudaEventDestroy(ctx->ev_join);
    if (ctx->scratch.ptr) cudaFree(ctx->scratch.ptr);
    if (ctx->stage.ptr) cudaFree(ctx->stage.ptr);
    for (void* p : ctx->retired) cudaFree(p);
    if (ctx->ragged_host) cudaFreeHost(ctx->ragged_host);
    if (ctx->ragged_dev) cudaFree(ctx->ragged_dev);
    if (ctx->ev_ragged) cudaEventDestroy(ctx->ev_ragged);
    if (ctx->status) cudaFree(ctx->status);
    if (ctx->counters) cudaFree(ctx->counters);
    delete ctx;
    return DKV_OK;
}

int dkv_context_reserve(dkv_context* ctx, int64_t max_rows, int nh_q, int nh_kv, int hidden) {
    DKV_REQUIRE(ctx != nullptr, "ctx is NULL");
    DKV_REQUIRE(max_rows > 0 && nh_q > 0 && nh_kv > 0 && nh_q % nh_kv == 0, "bad reserve sizes");
    DKV_CUDA(cudaSetDevice(ctx->device));
    ScratchPlan s = plan_scratch(ctx, max_rows, nh_q, nh_kv, hidden, hidden > 0, true);
    return ensure_buffer(ctx, &ctx->scratch, s.total, false, "scratch");
}

int dkv_context_set(dkv_context* ctx, const char* key, int value) {
    DKV_REQUIRE(ctx != nullptr && key != nullptr, "ctx / key is NULL");
    if (!strcmp(key, "attn_variant")) {
        DKV_REQUIRE(value >= -1 && value <= 2, "attn_variant must be -1 (automatic) or 0..2");
        ctx->attn_variant = value;
    } else if (!strcmp(key, "attn_ctas")) {
        DKV_REQUIRE(value >= 0 && value <= 65535, "attn_ctas out of range");
        ctx->attn_ctas = value;
    } else if (!strcmp(key, "check_coresidency")) {
        // The decode projection is built to run UNDER the 16-warp streaming kernels (same SMs, same time).  That
        // holds only while one CTA of each fits an SM's registers and shared memory together; a few registers more
        // in a streaming kernel silently turn the overlap into a sequence (+10 us on a 170 us step).
        DKV_CUDA(cudaSetDevice(ctx->device));
        cudaDeviceProp prop;
        DKV_CUDA(cudaGetDeviceProperties(&prop, ctx->device));
        cudaFuncAttributes pa, sa[2];
        DKV_CUDA(cudaFuncGetAttributes(&pa, proj_rope_decode_kernel));
        DKV_CUDA(cudaFuncGetAttributes(&sa[0], attn_partial_kernel<1, 16, 1>));
        DKV_CUDA(cudaFuncGetAttributes(&sa[1], attn_partial_mma8_kernel<16, 1>));
        const size_t stream_smem = attn_smem_bytes<1, 16, 1>();
        for (int i = 0; i < 2; ++i) {
            const long long regs = 512ll * sa[i].numRegs + 128ll * pa.numRegs;
            const size_t smem = stream_smem + sa[i].sharedSizeBytes + pd_smem_bytes(kPdMaxTokens) + pa.sharedSizeBytes + 2048;   // + 1 KB per CTA that the system reserves
            if (regs > prop.regsPerMultiprocessor || smem > prop.sharedMemPerMultiprocessor)
                return fail(DKV_ERR_UNSUPPORTED,
                            "the %s streaming kernel (%d registers, %zu B) and the decode projection (%d registers, %zu B) do not "
                            "fit one SM together (%lld of %d registers, %zu of %zu B)", i ? "tensor-core" : "CUDA-core",
                            sa[i].numRegs, stream_smem + sa[i].sharedSizeBytes, pa.numRegs,
                            pd_smem_bytes(kPdMaxTokens) + pa.sharedSizeBytes, regs, prop.regsPerMultiprocessor, smem,
                            static_cast<size_t>(prop.sharedMemPerMultiprocessor));
        }
        cudaFuncAttributes ga;
        DKV_CUDA(cudaFuncGetAttributes(&ga, proj_rope_gemv_kernel<kGvMaxTokens>));
        for (int i = 0; i < 2; ++i) {
            const long long regs = 512ll * sa[i].numRegs + 128ll * ga.numRegs;
            const size_t smem = stream_smem + sa[i].sharedSizeBytes + kGvSmemBudget + ga.sharedSizeBytes + 2048;
            if (regs > prop.regsPerMultiprocessor || smem > prop.sharedMemPerMultiprocessor)
                return fail(DKV_ERR_UNSUPPORTED,
                            "the %s streaming kernel and the matrix-vector projection do not fit one SM together "
                            "(%lld of %d registers, %zu of %zu B)", i ? "tensor-core" : "CUDA-core", regs,
                            prop.regsPerMultiprocessor, smem, static_cast<size_t>(prop.sharedMemPerMultiprocessor));
        }
    } else if (!strcmp(key, "attn_self_scan")) {
        ctx->attn_self_scan = value != 0;
    } else if (!strcmp(key, "proj_wide")) {
        ctx->proj_wide = value != 0;
    } else if (!strcmp(key, "proj_gemv")) {
        ctx->proj_gemv = value != 0;
    } else if (!strcmp(key, "proj_decode")) {
        DKV_REQUIRE(value >= -1 && value <= 1, "proj_decode must be -1, 0 or 1");
        ctx->proj_decode = value;
    } else if (!strcmp(key, "attn_mma8")) {
        ctx->attn_mma8 = value != 0;
    } else if (!strcmp(key, "attn_mma")) {
        DKV_REQUIRE(value >= -1 && value <= 1, "attn_mma must be -1, 0 or 1");
        ctx->attn_mma = value;
    } else if (!strcmp(key, "extend_pingpong")) {
        ctx->extend_pingpong = value != 0;
    } else if (!strcmp(key, "extend_rowwise")) {
        ctx->extend_rowwise = value ? 1 : 0;
    } else if (!strcmp(key, "wait_limit_ms")) {
        DKV_REQUIRE(value >= 1 && value <= 60000, "wait_limit_ms must be 1..60000");
        ctx->wait_limit_ms = value;
    } else if (!strcmp(key, "profile_attn")) {
        ctx->profile_attn = value ? 1 : 0;
    } else if (!strcmp(key, "attn_min_units")) {
        DKV_REQUIRE(value >= 1 && value <= 64, "attn_min_units must be 1..64");
        ctx->attn_min_units = static_cast<int>(value);
    } else if (!strcmp(key, "proj_split_k")) {
        DKV_REQUIRE(value >= 0 && value <= 256, "proj_split_k out of range");
        ctx->proj_split_k = value;
    } else {
        return fail(DKV_ERR_INVALID, "unknown tuning key '%s'", key);
    }
    return DKV_OK;
}

int dkv_read_status(dkv_context* ctx, unsigned int* status, int clear) {
    DKV_REQUIRE(ctx != nullptr && status != nullptr, "ctx / status is NULL");
    DKV_CUDA(cudaSetDevice(ctx->device));
    DKV_CUDA(cudaDeviceSynchronize());
    DKV_CUDA(cudaMemcpy(status, ctx->status, sizeof(unsigned int), cudaMemcpyDeviceToHost));
    if (clear && *status != 0) {
        DKV_CUDA(cudaMemset(ctx->status, 0, sizeof(unsigned int)));
        DKV_CUDA(cudaMemset(ctx->counters, 0, kMaxCounters * sizeof(unsigned int)));
    }
    return DKV_OK;
}

int dkv_profile_read(dkv_context* ctx, double* attn_ms_total, long long* attn_launches, long long* total_launches,
                     int reset) {
    DKV_REQUIRE(ctx != nullptr, "ctx is NULL");
    DKV_CUDA(cudaSetDevice(ctx->device));
    DKV_CUDA(cudaDeviceSynchronize());
    double ms = 0.0;
    for (size_t i = 0; i < ctx->attn_events_used; ++i) {
        float t = 0.f;
        DKV_CUDA(cudaEventElapsedTime(&t, ctx->attn_events[i].first, ctx->attn_events[i].second));
        ms += t;
    }
    if (attn_ms_total) *attn_ms_total = ms;
    if (attn_launches) *attn_launches = static_cast<long long>(ctx->attn_events_used);
    if (total_launches) *total_launches = ctx->launches;
    if (reset) {
        ctx->attn_events_used = 0;
        ctx->launches = 0;
    }
    return DKV_OK;
}

int dkv_layer_register(dkv_context* ctx, int layer_id, const dkv_layer_desc* desc) {
    DKV_REQUIRE(ctx != nullptr && desc != nullptr, "ctx / desc is NULL");
    DKV_CUDA(cudaSetDevice(ctx->device));
    LayerState L;
    int rc = build_layer(&L, desc);
    if (rc != DKV_OK) return rc;
    ctx->layers[layer_id] = L;
    return DKV_OK;
}

int dkv_layer_unregister(dkv_context* ctx, int layer_id) {
    DKV_REQUIRE(ctx != nullptr, "ctx is NULL");
    ctx->layers.erase(layer_id);
    return DKV_OK;
}

static int decode_impl(dkv_context* ctx, const dkv_decode_args* a, void* stream, dkv_exchange* ex) {
    DKV_REQUIRE(ctx != nullptr && a != nullptr, "ctx / args is NULL");
    auto it = ctx->layers.find(a->layer_id);
    if (it == ctx->layers.end())
        return fail(DKV_ERR_NOT_REGISTERED, "dkv_decode: layer %d not registered - call dkv_layer_register first",
                    a->layer_id);
    const LayerState& L = it->second;
    const int nh_kv = L.d.nh_kv;
    if (a->batch == 0) return DKV_OK;
    DKV_REQUIRE(a->batch > 0, "batch must be >= 0");
    DKV_REQUIRE(a->nh_q > 0 && a->nh_q % nh_kv == 0, "nh_q (%d) must be a multiple of nh_kv (%d)", a->nh_q, nh_kv);
    DKV_REQUIRE(a->q != nullptr && a->seq_lens != nullptr, "q / seq_lens must not be NULL");
    DKV_REQUIRE(a->out != nullptr || a->partial_out != nullptr || ex != nullptr, "out or partial_out must be given");
    DKV_REQUIRE(a->q_stride >= static_cast<int64_t>(a->nh_q) * 128 && a->q_stride % 8 == 0, "q_stride too small or unaligned");
    DKV_REQUIRE((reinterpret_cast<uintptr_t>(a->q) & 15) == 0, "q must be 16-byte aligned");
    if (a->out) {
        DKV_REQUIRE(a->out_stride >= static_cast<int64_t>(a->nh_q) * 128 && a->out_stride % 4 == 0, "out_stride too small or unaligned");
        DKV_REQUIRE((reinterpret_cast<uintptr_t>(a->out) & 7) == 0, "out must be 8-byte aligned");
    }
    const bool paged = a->page_table != nullptr;
    if (paged) DKV_REQUIRE(a->pt_stride > 0 && a->pt_rows >= 0, "pt_stride must be positive and pt_rows >= 0");
    else DKV_REQUIRE(L.d.row_stride > 0, "layer was registered without row_stride; pass a page_table");
    DKV_REQUIRE(a->new_mode >= DKV_NEW_NONE && a->new_mode <= DKV_NEW_GIVEN, "bad new_mode %d", a->new_mode);
    if (a->new_mode == DKV_NEW_PROJECT) {
        DKV_REQUIRE(L.has_weights, "layer %d has no projection weights registered", a->layer_id);
        DKV_REQUIRE(a->x != nullptr && (reinterpret_cast<uintptr_t>(a->x) & 15) == 0, "x must be a 16-byte aligned device pointer");
    }
    if (a->new_mode == DKV_NEW_GIVEN) DKV_REQUIRE(a->k_new && a->v_new, "k_new / v_new must not be NULL");
    DKV_CUDA(cudaSetDevice(ctx->device));
    cudaStream_t st = static_cast<cudaStream_t>(stream);

    const bool with_proj = a->new_mode == DKV_NEW_PROJECT;
    ScratchPlan sp = plan_scratch(ctx, a->batch, a->nh_q, nh_kv, L.d.hidden, with_proj, false);
    int rc = ensure_scratch(ctx, sp, st);
    if (rc != DKV_OK) return rc;
    uint8_t* base = ctx->scratch.ptr;
    int* cum = reinterpret_cast<int*>(base + sp.cum);
    int* tok_pos = reinterpret_cast<int*>(base + sp.tok_pos);
    int* tok_slot = reinterpret_cast<int*>(base + sp.tok_slot);
    __nv_bfloat16* kv_new = reinterpret_cast<__nv_bfloat16*>(base + sp.kv_new);
    const int n_new = a->new_mode == DKV_NEW_NONE ? 0 : 1;

    PrepParams prep{};
    prep.seq_lens = a->seq_lens;
    prep.batch = a->batch;
    prep.n_new = n_new;
    prep.cum_tiles = cum;
    prep.tok_pos = tok_pos;
    prep.tok_slot = tok_slot;
    prep.page_table = a->page_table;
    prep.row_map = a->row_map;
    prep.pos_offset = a->pos_offset;
    prep.pt_stride = a->pt_stride;
    prep.pt_rows = a->pt_rows;
    prep.status = ctx->status;
    prep.page_size = L.d.page_size;
    prep.page_shift = L.page_shift;
    prep.row_stride = L.d.row_stride;
    prep.save = a->save_kv_cache;
    if (a->new_mode == DKV_NEW_PROJECT) {
        // The projection depends neither on the streamed attention nor on the prep kernel (it works out the new
        // tokens' positions and slots itself): it runs on the context's side stream, forked before prep and
        // joined before the merge, so a short step has it off the critical path from the start.
        DKV_CUDA(cudaEventRecord(ctx->ev_fork, st));
        DKV_CUDA(cudaStreamWaitEvent(ctx->side, ctx->ev_fork, 0));
    }
    // Small batches need no prep launch: the streaming and merge kernels scan the lengths themselves, and the
    // projection places its tokens itself.  Caller-given K/V rows still take their slots from the prep kernel.
    const bool self_scan = ctx->attn_self_scan != 0 && a->batch <= kSelfScanMax && a->new_mode != DKV_NEW_GIVEN;
    if (!self_scan) {
        attn_prep_kernel<<<1, 256, 0, st>>>(prep);
        DKV_CUDA(cudaGetLastError());
        ctx->launches += 1;
    }
    ctx->launches += (a->new_mode == DKV_NEW_GIVEN ? 1 : 0);
    if (a->new_mode == DKV_NEW_PROJECT) {
        const int g_total = a->nh_q / nh_kv;
        bool rows_on_host = L.pool_on_host;              // where the streaming kernel will read from
        if (a->kv_source_layer != 0) {
            auto its = ctx->layers.find(a->kv_source_layer);
            if (its != ctx->layers.end()) rows_on_host = its->second.pool_on_host;
        }
        // Forms of the streaming kernel that leave the projection registers and shared memory on every SM: the
        // 16-warp CUDA-core form (one query head per KV head) and the 16-warp tensor-core form for up to 8.
        const bool mma_form = use_mma(ctx, g_total, rows_on_host);
        const int G_form = choose_g(ctx, g_total, rows_on_host);
        const bool beside = a->batch > 0 &&
                            ((!mma_form && G_form == 1 && effective_variant(ctx, 1) == 2) ||
                             (mma_form && G_form <= 8 && ctx->attn_mma8 != 0 && (ctx->attn_variant < 0 || ctx->attn_variant == 2)));
        DecodePlace place{};
        place.seq_lens = a->seq_lens;
        place.page_table = a->page_table;
        place.row_map = a->row_map;
        place.pos_offset = a->pos_offset;
        place.pt_stride = a->pt_stride;
        place.pt_rows = a->pt_rows;
        place.page_size = L.d.page_size;
        place.page_shift = L.page_shift;
        place.row_stride = L.d.row_stride;
        place.save = a->save_kv_cache;
        rc = launch_projection(ctx, L, a->x, a->batch, nullptr, nullptr, a->save_kv_cache != 0, kv_new,
                               reinterpret_cast<float*>(base + sp.splitk), ctx->side, beside, nullptr, nullptr, 0, &place);
        if (rc != DKV_OK) return rc;
        DKV_CUDA(cudaEventRecord(ctx->ev_join, ctx->side));
    } else if (a->new_mode == DKV_NEW_GIVEN) {
        const long long warps = static_cast<long long>(a->batch) * nh_kv;
        store_new_kv_kernel<<<static_cast<int>((warps + 3) / 4), 128, 0, st>>>(
            static_cast<const __nv_bfloat16*>(a->k_new), static_cast<const __nv_bfloat16*>(a->v_new), a->batch, nh_kv,
            tok_slot, static_cast<__nv_bfloat16*>(L.k_dev), static_cast<__nv_bfloat16*>(L.v_dev), L.d.n_slots, kv_new,
            ctx->status);
        DKV_CUDA(cudaGetLastError());
    }

    AttnParams ap{};
    ap.q = static_cast<const __nv_bfloat16*>(a->q);
    ap.q_stride = a->q_stride;
    // The past rows are read from the layer's own pool, or from a copy of them registered as another layer.
    const LayerState* Lsrc = &L;
    bool src_paged = paged;
    ap.page_table = a->page_table;
    ap.row_map = a->row_map;
    ap.pt_stride = a->pt_stride;
    ap.pt_rows = a->pt_rows;
    if (a->kv_source_layer != 0) {
        auto its = ctx->layers.find(a->kv_source_layer);
        if (its == ctx->layers.end())
            return fail(DKV_ERR_NOT_REGISTERED, "dkv_decode: kv_source_layer %d not registered", a->kv_source_layer);
        Lsrc = &its->second;
        DKV_REQUIRE(Lsrc->d.nh_kv == nh_kv, "kv_source_layer has %d KV heads, the layer %d", Lsrc->d.nh_kv, nh_kv);
        src_paged = a->src_page_table != nullptr;
        if (src_paged) DKV_REQUIRE(a->src_pt_stride > 0, "src_pt_stride must be positive");
        else DKV_REQUIRE(Lsrc->d.row_stride > 0, "kv_source_layer was registered without row_stride; pass src_page_table");
        ap.page_table = a->src_page_table;
        ap.row_map = a->src_row_map;
        ap.pt_stride = a->src_pt_stride;
        ap.pt_rows = 0;
    }
    ap.seq_lens = a->seq_lens;
    ap.cum_tiles = cum;
    ap.partials = reinterpret_cast<float*>(base + sp.partials);
    ap.status = ctx->status;
    ap.batch = a->batch;
    ap.nh_q = a->nh_q;
    ap.nh_kv = nh_kv;
    ap.g_total = a->nh_q / nh_kv;
    ap.page_size = Lsrc->d.page_size;
    ap.page_shift = Lsrc->page_shift;
    ap.rows_per_box = Lsrc->rows_per_box;
    ap.row_stride = Lsrc->d.row_stride;
    ap.n_new = n_new;
    ap.self_scan = self_scan ? 1 : 0;
    ap.scale_log2 = a->softmax_scale * 1.4426950408889634f;
    MergeParams mp{};
    mp.kv_new = n_new ? kv_new : nullptr;
    mp.out = static_cast<__nv_bfloat16*>(a->out);
    mp.out_stride = a->out_stride;
    mp.lse = a->lse_out;
    mp.part_out = a->partial_out;
    if (ex != nullptr) {
        const int parity = static_cast<int>(ex->steps & 1ull);
        mp.x_world = ex->world;
        mp.x_rank = ex->rank;
        mp.x_tag = static_cast<unsigned int>(ex->steps % 0xfffffffeull) + 1u;
        mp.x_max_rows = ex->max_rows;
        for (int r = 0; r < ex->world; ++r) {
            mp.x_part[r] = ex->part[r] + parity * ex->half_floats;
            mp.x_count[r] = ex->count[r] + parity * kMaxExchangeRanks;
        }
    }
    return launch_attention(ctx, *Lsrc, ap, src_paged, mp, st, a->new_mode == DKV_NEW_PROJECT ? ctx->ev_join : nullptr);
}

int dkv_decode(dkv_context* ctx, const dkv_decode_args* a, void* stream) { return decode_impl(ctx, a, stream, nullptr); }

int dkv_exchange_create(dkv_context* ctx, int rank, int world, int64_t max_rows, dkv_exchange** out) {
    DKV_REQUIRE(ctx != nullptr && out != nullptr, "ctx / out is NULL");
    DKV_REQUIRE(world >= 1 && world <= kMaxExchangeRanks && rank >= 0 && rank < world, "bad rank %d / world %d (at most %d ranks)",
                rank, world, kMaxExchangeRanks);
    DKV_REQUIRE(max_rows > 0, "max_rows must be positive");
    DKV_CUDA(cudaSetDevice(ctx->device));
    dkv_exchange* ex = new dkv_exchange();
    ex->ctx = ctx;
    ex->rank = rank;
    ex->world = world;
    ex->max_rows = max_rows;
    ex->half_floats = static_cast<size_t>(world) * max_rows * kPartialStride;
    ex->part_bytes = align256(2 * ex->half_floats * sizeof(float));
    cudaError_t e = cudaMalloc(&ex->local, ex->part_bytes + 256);
    if (e == cudaSuccess) e = cudaMemset(ex->local, 0, ex->part_bytes + 256);
    if (e != cudaSuccess) {
        delete ex;
        return fail(DKV_ERR_CUDA, "exchange buffer allocation failed: %s", cudaGetErrorString(e));
    }
    ex->part[rank] = reinterpret_cast<float*>(ex->local);
    ex->count[rank] = reinterpret_cast<unsigned int*>(ex->local + ex->part_bytes);
    *out = ex;
    return DKV_OK;
}

int dkv_exchange_handle(dkv_exchange* ex, void* handle_out_64_bytes) {
    DKV_REQUIRE(ex != nullptr && handle_out_64_bytes != nullptr, "NULL argument");
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
    DKV_CUDA(cudaSetDevice(ex->ctx->device));
    cudaIpcMemHandle_t h;
    DKV_CUDA(cudaIpcGetMemHandle(&h, ex->local));
    memcpy(handle_out_64_bytes, &h, sizeof(h));
    return DKV_OK;
}

int dkv_exchange_connect(dkv_exchange* ex, int peer_rank, const void* handle_64_bytes) {
    DKV_REQUIRE(ex != nullptr && handle_64_bytes != nullptr, "NULL argument");
    DKV_REQUIRE(peer_rank >= 0 && peer_rank < ex->world && peer_rank != ex->rank, "bad peer rank %d", peer_rank);
    DKV_CUDA(cudaSetDevice(ex->ctx->device));
    cudaIpcMemHandle_t h;
    memcpy(&h, handle_64_bytes, sizeof(h));
    void* base = nullptr;
    DKV_CUDA(cudaIpcOpenMemHandle(&base, h, cudaIpcMemLazyEnablePeerAccess));
    ex->opened[peer_rank] = base;
    ex->part[peer_rank] = reinterpret_cast<float*>(base);
    ex->count[peer_rank] = reinterpret_cast<unsigned int*>(static_cast<uint8_t*>(base) + ex->part_bytes);
    return DKV_OK;
}

int dkv_exchange_connect_ptr(dkv_exchange* ex, int peer_rank, void* peer_base) {
    DKV_REQUIRE(ex != nullptr && peer_base != nullptr, "NULL argument");
    DKV_REQUIRE(peer_rank >= 0 && peer_rank < ex->world && peer_rank != ex->rank, "bad peer rank %d", peer_rank);
    ex->part[peer_rank] = reinterpret_cast<float*>(peer_base);
    ex->count[peer_rank] = reinterpret_cast<unsigned int*>(static_cast<uint8_t*>(peer_base) + ex->part_bytes);
    return DKV_OK;
}

int dkv_exchange_base(dkv_exchange* ex, void** base_out) {
    DKV_REQUIRE(ex != nullptr && base_out != nullptr, "NULL argument");
    *base_out = ex->local;
    return DKV_OK;
}

int dkv_exchange_destroy(dkv_exchange* ex) {
    if (!ex) return DKV_OK;
    cudaSetDevice(ex->ctx->device);
    cudaDeviceSynchronize();
    for (int r = 0; r < ex->world; ++r)
        if (ex->opened[r]) cudaIpcCloseMemHandle(ex->opened[r]);
    if (ex->local) cudaFree(ex->local);
    delete ex;
    return DKV_OK;
}

int dkv_decode_exchange(dkv_context* ctx, dkv_exchange* ex, const dkv_decode_args* a, void* out, float* lse,
                        void* stream) {
    DKV_REQUIRE(ctx != nullptr && ex != nullptr && a != nullptr && out != nullptr, "NULL argument");
    DKV_REQUIRE(ex->ctx == ctx, "the exchange belongs to another context");
    for (int r = 0; r < ex->world; ++r)
        DKV_REQUIRE(ex->part[r] != nullptr, "exchange: rank %d is not connected", r);
    const long long rows = static_cast<long long>(a->batch) * a->nh_q;
    DKV_REQUIRE(rows > 0 && rows <= ex->max_rows, "batch * nh_q (%lld) exceeds the exchange's max_rows (%lld)", rows,
                ex->max_rows);
    dkv_decode_args local = *a;
    local.out = nullptr;
    local.partial_out = nullptr;
    local.lse_out = nullptr;
    int rc = decode_impl(ctx, &local, stream, ex);
    if (rc != DKV_OK) return rc;
    // Why two halves are enough: a rank's consumer kernel of step n runs after its own producer of step n (same
    // stream), and returns only when every rank's step-n records have landed here.  So when rank A issues stores
    // of step n+1, every rank has finished PRODUCING step n, and A has finished consuming it; a slower rank B may
    // still be consuming step n - from the half of parity n, which A's step-n+1 stores do not touch.  A cannot
    // reach step n+2 before B has produced step n+1, which B does only after its step-n consumer.
    const int parity = static_cast<int>(ex->steps & 1ull);
    ExchangeMergeParams ep{};
    ep.parts = ex->part[ex->rank] + parity * ex->half_floats;
    ep.count = ex->count[ex->rank] + parity * kMaxExchangeRanks;
    ep.tag = static_cast<unsigned int>(ex->steps % 0xfffffffeull) + 1u;
    for (int r = 0; r < ex->world; ++r) {
        ex->expected[parity][r] += static_cast<unsigned int>(rows);   // every rank delivers `rows` records per step
        ep.expected[r] = ex->expected[parity][r];
    }
    ex->steps += 1;
    ep.world = ex->world;
    ep.max_rows = ex->max_rows;
    ep.rows = rows;
    ep.out = static_cast<__nv_bfloat16*>(out);
    ep.lse = lse;
    ep.status = ctx->status;
    ep.wait_limit_ns = static_cast<unsigned long long>(ctx->wait_limit_ms) * 1000000ull;
    merge_exchange_kernel<<<static_cast<int>((rows + 3) / 4), 128, 0, static_cast<cudaStream_t>(stream)>>>(ep);
    DKV_CUDA(cudaGetLastError());
    ctx->launches += 1;
    return DKV_OK;
}

int dkv_merge_partials(dkv_context* ctx, const float* parts, int nranks, int64_t rows, void* out, float* lse,
                       void* stream) {
    DKV_REQUIRE(ctx != nullptr && parts != nullptr && out != nullptr, "NULL argument");
    DKV_REQUIRE(nranks > 0 && rows > 0, "nranks and rows must be positive");
    DKV_CUDA(cudaSetDevice(ctx->device));
    merge_rank_partials_kernel<<<static_cast<int>((rows + 3) / 4), 128, 0, static_cast<cudaStream_t>(stream)>>>(
        parts, nranks, rows, static_cast<__nv_bfloat16*>(out), lse);
    DKV_CUDA(cudaGetLastError());
    return DKV_OK;
}

// Shared by the eager and the graph-safe extend entry points.
static int run_extend(dkv_context* ctx, const LayerState& L, const void* X, const void* Q, void* O, int B, int S_new,
                      int nh_q, float scale, int is_causal, int seqlen_past, const int32_t* n_past_blocks_dev,
                      int q_pos_start, const int32_t* row_map, cudaStream_t st, const int32_t* page_table = nullptr,
                      long long pt_stride = 0) {
    const int nh_kv = L.d.nh_kv;
    const int64_t rows = static_cast<int64_t>(B) * S_new;
    const bool qrot = (L.d.cos_sin != nullptr && q_pos_start >= 0);
    const bool project = (X != nullptr);              // nullptr: the new rows are in the pool already
    const bool paged = (page_table != nullptr);
    // Host pool, length known on the host, more than one query tile: stage the rows in HBM once.  A paged pool is
    // always staged: the gather through the page table makes the rows contiguous for the tensor-core kernel.
    const int s_total_host = seqlen_past + S_new;
    const bool tensor_path = !ctx->extend_rowwise || paged;
    const bool stage = paged || (!ctx->extend_rowwise && L.pool_on_host && n_past_blocks_dev == nullptr &&
                                 static_cast<long long>(S_new) * (nh_q / nh_kv) > kExtTile);
    // With a staging copy the new rows are projected straight into it (the attention reads them there) and reach
    // the host pool from the copy on the side stream, while the attention runs.
    const bool proj_to_stage = project && stage;
    // Copy engines instead of SM loads/stores where the host knows the rows: request b in pool row b, contiguous.
    const bool dma_rows = stage && !paged && L.pool_on_host && row_map == nullptr;
    const size_t row_bytes = static_cast<size_t>(nh_kv) * 256;
    const size_t stage_bytes = stage ? static_cast<size_t>(B) * s_total_host * nh_kv * 256 : 0;
    ScratchPlan sp = plan_scratch(ctx, rows, nh_q, nh_kv, L.d.hidden, project, qrot, stage_bytes);
    int rc = ensure_scratch(ctx, sp, st);
    if (rc != DKV_OK) return rc;
    uint8_t* base = ctx->scratch.ptr;
    int* cum = reinterpret_cast<int*>(base + sp.cum);
    int* tok_pos = reinterpret_cast<int*>(base + sp.tok_pos);
    int* tok_slot = reinterpret_cast<int*>(base + sp.tok_slot);
    int* vseq = reinterpret_cast<int*>(base + sp.vseq);
    int* vrow = reinterpret_cast<int*>(base + sp.vrow);
    if (paged && (project || n_past_blocks_dev != nullptr))
        return fail(DKV_ERR_INVALID, "a paged pool is supported for attention over stored rows with a host-side length only");

    extend_prep_kernel<<<static_cast<int>((rows + 255) / 256), 256, 0, st>>>(
        B, S_new, seqlen_past, n_past_blocks_dev, is_causal, row_map, L.d.row_stride, vseq, vrow, tok_pos, tok_slot,
        s_total_host, proj_to_stage ? cum : nullptr);
    DKV_CUDA(cudaGetLastError());
    ctx->launches += 1;
    if (!tensor_path) {
        // Only the row-streamed path walks tile cursors: prefix sum of the virtual requests' tile counts.
        PrepParams prep{};
        prep.seq_lens = vseq;
        prep.batch = static_cast<int>(rows);
        prep.n_new = 0;
        prep.cum_tiles = cum;
        attn_prep_kernel<<<1, 256, 0, st>>>(prep);
        DKV_CUDA(cudaGetLastError());
        ctx->launches += 1;
    }
    uint4* stage_k = stage ? reinterpret_cast<uint4*>(ctx->stage.ptr + sp.stage_k) : nullptr;
    uint4* stage_v = stage ? reinterpret_cast<uint4*>(ctx->stage.ptr + sp.stage_v) : nullptr;
    if (project) {
        rc = launch_projection(ctx, L, X, static_cast<int>(rows), tok_pos, proj_to_stage ? cum : tok_slot, true, nullptr,
                               reinterpret_cast<float*>(base + sp.splitk), st, false, proj_to_stage ? stage_k : nullptr,
                               proj_to_stage ? stage_v : nullptr, static_cast<long long>(B) * s_total_host);
        if (rc != DKV_OK) return rc;
        if (proj_to_stage) {
            DKV_CUDA(cudaEventRecord(ctx->ev_fork, st));
            DKV_CUDA(cudaStreamWaitEvent(ctx->side, ctx->ev_fork, 0));
            if (dma_rows) {
                // Rows known on the host (request b lives in pool row b): one copy-engine transfer per request and tensor.
                for (int b = 0; b < B; ++b) {
                    const size_t src = (static_cast<size_t>(b) * s_total_host + seqlen_past) * row_bytes;
                    const size_t dst = (static_cast<size_t>(b) * L.d.row_stride + seqlen_past) * row_bytes;
                    DKV_CUDA(cudaMemcpyAsync(static_cast<uint8_t*>(L.d.k_pool) + dst, reinterpret_cast<uint8_t*>(stage_k) + src,
                                             static_cast<size_t>(S_new) * row_bytes, cudaMemcpyDeviceToHost, ctx->side));
                    DKV_CUDA(cudaMemcpyAsync(static_cast<uint8_t*>(L.d.v_pool) + dst, reinterpret_cast<uint8_t*>(stage_v) + src,
                                             static_cast<size_t>(S_new) * row_bytes, cudaMemcpyDeviceToHost, ctx->side));
                }
            } else {
                unstage_rows_kernel<<<ctx->sm_count * 2, 256, 0, ctx->side>>>(
                    static_cast<uint4*>(L.k_dev), static_cast<uint4*>(L.v_dev), stage_k, stage_v, cum, tok_slot, rows, nh_kv * 16,
                    L.d.n_slots, ctx->status);
                DKV_CUDA(cudaGetLastError());
                ctx->launches += 1;
            }
            DKV_CUDA(cudaEventRecord(ctx->ev_join, ctx->side));
        }
    }
    const __nv_bfloat16* q_use = static_cast<const __nv_bfloat16*>(Q);
    if (qrot) {
        __nv_bfloat16* q_rot = reinterpret_cast<__nv_bfloat16*>(base + sp.q_rot);
        const long long total = rows * nh_q * 64;
        rope_q_kernel<<<static_cast<int>((total + 255) / 256), 256, 0, st>>>(q_use, q_rot, B, S_new, nh_q, L.d.cos_sin,
                                                                           L.d.max_pos, q_pos_start, ctx->status);
        DKV_CUDA(cudaGetLastError());
        q_use = q_rot;
    }
    if (tensor_path) {
        // Tensor-core path: 128 query rows per CTA = G query heads x 128/G tokens of one KV head.
        const int g_total = nh_q / nh_kv;
        int G = 1;
        while (G < 128 && g_total % (2 * G) == 0) G *= 2;
        const int nsub = g_total / G;
        const int TQ = kExtTile / G;
        CUtensorMap tmQ;
        rc = encode_tile_map(&tmQ, q_use, rows, nh_q, G, TQ);
        if (rc != DKV_OK) return rc;
        const CUtensorMap* tmK = &L.tmK_128;
        const CUtensorMap* tmV = &L.tmV_128;
        CUtensorMap tmKs, tmVs;
        const int32_t* ext_rows = row_map;
        long long ext_stride = L.d.row_stride;
        if (stage) {
            uint4* ks = stage_k;
            uint4* vs = stage_v;
            if (dma_rows) {
                const int n = proj_to_stage ? seqlen_past : s_total_host;
                for (int b = 0; b < B && n > 0; ++b) {
                    const size_t src = static_cast<size_t>(b) * L.d.row_stride * row_bytes;
                    const size_t dst = static_cast<size_t>(b) * s_total_host * row_bytes;
                    DKV_CUDA(cudaMemcpyAsync(reinterpret_cast<uint8_t*>(ks) + dst, static_cast<const uint8_t*>(L.d.k_pool) + src,
                                             static_cast<size_t>(n) * row_bytes, cudaMemcpyHostToDevice, st));
                    DKV_CUDA(cudaMemcpyAsync(reinterpret_cast<uint8_t*>(vs) + dst, static_cast<const uint8_t*>(L.d.v_pool) + src,
                                             static_cast<size_t>(n) * row_bytes, cudaMemcpyHostToDevice, st));
                }
            } else {
                stage_rows_kernel<<<ctx->sm_count * 8, 256, 0, st>>>(ks, vs, static_cast<const uint4*>(L.k_dev),
                                                                     static_cast<const uint4*>(L.v_dev), row_map,
                                                                     L.d.row_stride, B, s_total_host, nh_kv * 16, page_table,
                                                                     pt_stride, L.page_shift, proj_to_stage ? seqlen_past : -1);
                DKV_CUDA(cudaGetLastError());
                ctx->launches += 1;
            }
            const int64_t srows = static_cast<int64_t>(B) * s_total_host;
            if ((rc = encode_tile_map(&tmKs, ks, srows, nh_kv, 1, kExtTile)) != DKV_OK) return rc;
            if ((rc = encode_tile_map(&tmVs, vs, srows, nh_kv, 1, kExtTile)) != DKV_OK) return rc;
            tmK = &tmKs;
            tmV = &tmVs;
            ext_rows = nullptr;
            ext_stride = s_total_host;
        }
        ExtendParams ep{};
        ep.vrow = ext_rows;
        ep.n_past_blocks = n_past_blocks_dev;
        ep.seqlen_past = seqlen_past;
        ep.S_new = S_new;
        ep.nh_q = nh_q;
        ep.nh_kv = nh_kv;
        ep.G = G;
        ep.g_total = g_total;
        ep.nsub = nsub;
        ep.row_stride = ext_stride;
        ep.is_causal = is_causal;
        ep.scale_log2 = scale * 1.4426950408889634f;
        ep.out = static_cast<__nv_bfloat16*>(O);
        ep.status = ctx->status;
        if (ctx->extend_pingpong != 0) {
            // Head slots vary fastest so that the longest (latest) query tiles of ALL heads are dispatched first.
            dim3 grid(nh_kv * nsub, (S_new + 2 * TQ - 1) / (2 * TQ), B);
            extend_attn_pp_kernel<<<grid, kPpThreads, kPpSmem, st>>>(tmQ, *tmK, *tmV, ep);
        } else {
            dim3 grid((S_new + TQ - 1) / TQ, nh_kv * nsub, B);
            extend_attn_kernel<<<grid, 128, kExtSmem + 1024, st>>>(tmQ, *tmK, *tmV, ep);
        }
        DKV_CUDA(cudaGetLastError());
        ctx->launches += 1;
        if (proj_to_stage) DKV_CUDA(cudaStreamWaitEvent(st, ctx->ev_join, 0));   // the pool holds the new rows when the call's work is done
        return DKV_OK;
    }
    AttnParams ap{};
    ap.q = q_use;
    ap.q_stride = static_cast<long long>(nh_q) * 128;
    ap.page_table = nullptr;
    ap.row_map = vrow;
    ap.seq_lens = vseq;
    ap.cum_tiles = cum;
    ap.partials = reinterpret_cast<float*>(base + sp.partials);
    ap.status = ctx->status;
    ap.batch = static_cast<int>(rows);
    ap.nh_q = nh_q;
    ap.nh_kv = nh_kv;
    ap.g_total = nh_q / nh_kv;
    ap.page_size = 1;
    ap.page_shift = 0;
    ap.rows_per_box = kTileTokens;
    ap.row_stride = L.d.row_stride;
    ap.n_new = 0;
    ap.scale_log2 = scale * 1.4426950408889634f;
    MergeParams mp{};
    mp.out = static_cast<__nv_bfloat16*>(O);
    mp.out_stride = static_cast<long long>(nh_q) * 128;
    return launch_attention(ctx, L, ap, false, mp, st);
}

int dkv_smpv2_fwd(dkv_context* ctx, const void* X, const void* Wk, const void* Wv, const void* Q, void* K_cpu,
                  void* V_cpu, const float* cos_sin, int max_pos, int B, int S_new, int H, int nh_q, int nh_kv,
                  int S_total, float softmax_scale, int is_causal, int seqlen_past, int q_pos_start, void* O,
                  void* stream) {
    DKV_REQUIRE(ctx != nullptr, "ctx is NULL");
    DKV_REQUIRE(X && Wk && Wv && Q && K_cpu && V_cpu && O, "NULL tensor pointer");
    DKV_REQUIRE(B > 0 && S_new > 0 && H > 0 && nh_q > 0 && nh_kv > 0, "sizes must be positive");
    // directkv/kernel/smpv2_extension.cu:176-178
    DKV_REQUIRE(S_total == seqlen_past + S_new, "K_cpu S_total (%d) != seqlen_past (%d) + S_new (%d)", S_total, seqlen_past, S_new);
    // directkv/kernel/smpv2_extension.cu:606-609
    DKV_REQUIRE(nh_q % nh_kv == 0, "Q.size(2) (NH_q=%d) must be a multiple of Wk.size(0) (NH_kv=%d)", nh_q, nh_kv);
    DKV_REQUIRE(seqlen_past >= 0, "seqlen_past must be >= 0");
    DKV_REQUIRE(H % 64 == 0, "hidden size (%d) must be a multiple of 64", H);
    DKV_REQUIRE((reinterpret_cast<uintptr_t>(X) & 15) == 0 && (reinterpret_cast<uintptr_t>(Q) & 15) == 0 &&
                    (reinterpret_cast<uintptr_t>(Wk) & 15) == 0 && (reinterpret_cast<uintptr_t>(Wv) & 15) == 0,
                "X, Q, Wk, Wv must be 16-byte aligned");
    DKV_CUDA(cudaSetDevice(ctx->device));
    dkv_layer_desc d{};
    d.k_pool = K_cpu;
    d.v_pool = V_cpu;
    d.n_slots = static_cast<int64_t>(B) * S_total;
    d.nh_kv = nh_kv;
    d.page_size = 1;
    d.row_stride = S_total;
    d.wk = Wk;
    d.wv = Wv;
    d.hidden = H;
    d.cos_sin = cos_sin;
    d.max_pos = max_pos;
    LayerState L;
    int rc = build_layer(&L, &d);
    if (rc != DKV_OK) return rc;
    return run_extend(ctx, L, X, Q, O, B, S_new, nh_q, softmax_scale, is_causal, seqlen_past, nullptr, q_pos_start,
                      nullptr, static_cast<cudaStream_t>(stream));
}

int dkv_smpv2_fwd_graph(dkv_context* ctx, int layer_id, const void* X_pad, const void* Q_pad, void* O_out,
                        const int32_t* n_past_blocks_dev, int B, int S_new, int nh_q, float softmax_scale,
                        int is_causal, const int32_t* req_pool_indices, void* stream) {
    DKV_REQUIRE(ctx != nullptr, "ctx is NULL");
    auto it = ctx->layers.find(layer_id);
    if (it == ctx->layers.end())
        return fail(DKV_ERR_NOT_REGISTERED, "smpv2_fwd_graph: layer %d not initialized - call smpv2_init_tma first", layer_id);
    const LayerState& L = it->second;
    DKV_REQUIRE(X_pad && Q_pad && O_out && n_past_blocks_dev, "NULL tensor pointer");
    DKV_REQUIRE(B > 0 && S_new > 0 && nh_q > 0 && nh_q % L.d.nh_kv == 0, "bad sizes");
    DKV_REQUIRE(L.has_weights, "layer %d has no projection weights registered", layer_id);
    DKV_REQUIRE(L.d.row_stride > 0, "layer %d was registered without row_stride", layer_id);
    DKV_CUDA(cudaSetDevice(ctx->device));
    return run_extend(ctx, L, X_pad, Q_pad, O_out, B, S_new, nh_q, softmax_scale, is_causal, 0, n_past_blocks_dev, -1,
                      req_pool_indices, static_cast<cudaStream_t>(stream));
}

int dkv_extend(dkv_context* ctx, int layer_id, const void* X, const void* Q, void* O, int B, int S_new, int nh_q,
               float softmax_scale, int is_causal, int seqlen_past, int q_pos_start, const int32_t* row_map,
               void* stream) {
    DKV_REQUIRE(ctx != nullptr, "ctx is NULL");
    auto it = ctx->layers.find(layer_id);
    if (it == ctx->layers.end())
        return fail(DKV_ERR_NOT_REGISTERED, "dkv_extend: layer %d not registered - call dkv_layer_register first", layer_id);
    const LayerState& L = it->second;
    DKV_REQUIRE(X && Q && O, "NULL tensor pointer");
    DKV_REQUIRE(B > 0 && S_new > 0 && nh_q > 0 && nh_q % L.d.nh_kv == 0, "bad sizes");
    DKV_REQUIRE(seqlen_past >= 0, "seqlen_past must be >= 0");
    DKV_REQUIRE(L.has_weights, "layer %d has no projection weights registered", layer_id);
    DKV_REQUIRE(L.d.row_stride > 0, "layer %d was registered without row_stride", layer_id);
    DKV_REQUIRE(seqlen_past + S_new <= L.d.row_stride, "seqlen_past + S_new (%d) exceeds the pool row (%lld)",
                seqlen_past + S_new, (long long)L.d.row_stride);
    DKV_CUDA(cudaSetDevice(ctx->device));
    return run_extend(ctx, L, X, Q, O, B, S_new, nh_q, softmax_scale, is_causal, seqlen_past, nullptr, q_pos_start,
                      row_map, static_cast<cudaStream_t>(stream));
}

int dkv_extend_attend(dkv_context* ctx, int layer_id, const void* Q, void* O, int B, int S_new, int nh_q,
                      float softmax_scale, int is_causal, int seqlen_past, const int32_t* row_map,
                      const int32_t* page_table, int64_t pt_stride, void* stream) {
    DKV_REQUIRE(ctx != nullptr, "ctx is NULL");
    auto it = ctx->layers.find(layer_id);
    if (it == ctx->layers.end())
        return fail(DKV_ERR_NOT_REGISTERED, "dkv_extend_attend: layer %d not registered - call dkv_layer_register first",
                    layer_id);
    const LayerState& L = it->second;
    DKV_REQUIRE(Q && O, "NULL tensor pointer");
    DKV_REQUIRE(B > 0 && S_new > 0 && nh_q > 0 && nh_q % L.d.nh_kv == 0, "bad sizes");
    DKV_REQUIRE(seqlen_past >= 0, "seqlen_past must be >= 0");
    if (page_table != nullptr) {
        DKV_REQUIRE(pt_stride > 0, "pt_stride must be positive with a page table");
        DKV_REQUIRE(((static_cast<int64_t>(seqlen_past) + S_new - 1) >> L.page_shift) < pt_stride,
                    "seqlen_past + S_new (%d) does not fit a page-table row of %lld pages", seqlen_past + S_new,
                    (long long)pt_stride);
    } else {
        DKV_REQUIRE(L.d.row_stride > 0, "layer %d was registered without row_stride and no page table was given", layer_id);
        DKV_REQUIRE(seqlen_past + S_new <= L.d.row_stride, "seqlen_past + S_new (%d) exceeds the pool row (%lld)",
                    seqlen_past + S_new, (long long)L.d.row_stride);
    }
    DKV_CUDA(cudaSetDevice(ctx->device));
    return run_extend(ctx, L, nullptr, Q, O, B, S_new, nh_q, softmax_scale, is_causal, seqlen_past, nullptr, -1, row_map,
                      static_cast<cudaStream_t>(stream), page_table, pt_stride);
}

// Grows the pinned host mirror and the device copy of the ragged-extend metadata (outside graph capture).
static int ensure_ragged(dkv_context* ctx, size_t ints) {
    if (ctx->ev_ragged == nullptr) DKV_CUDA(cudaEventCreateWithFlags(&ctx->ev_ragged, cudaEventDisableTiming));
    if (ints <= ctx->ragged_ints) return DKV_OK;
    if (ctx->ragged_pending) {
        DKV_CUDA(cudaEventSynchronize(ctx->ev_ragged));
        ctx->ragged_pending = false;
    }
    DKV_CUDA(cudaDeviceSynchronize());   // earlier launches may still read the old device copy
    if (ctx->ragged_host) cudaFreeHost(ctx->ragged_host);
    if (ctx->ragged_dev) cudaFree(ctx->ragged_dev);
    ctx->ragged_host = nullptr;
    ctx->ragged_dev = nullptr;
    ctx->ragged_ints = 0;
    const size_t want = ints + ints / 2 + 1024;
    DKV_CUDA(cudaHostAlloc(reinterpret_cast<void**>(&ctx->ragged_host), want * sizeof(int), cudaHostAllocDefault));
    DKV_CUDA(cudaMalloc(reinterpret_cast<void**>(&ctx->ragged_dev), want * sizeof(int)));
    ctx->ragged_ints = want;
    return DKV_OK;
}

int dkv_extend_ragged(dkv_context* ctx, int layer_id, const void* X, const void* Q, void* O, int B,
                      const int32_t* s_new_host, const int32_t* past_host, const int32_t* rows_host, int nh_q,
                      float softmax_scale, int is_causal, const int32_t* page_table, int64_t pt_stride, void* stream) {
    DKV_REQUIRE(ctx != nullptr, "ctx is NULL");
    auto it = ctx->layers.find(layer_id);
    if (it == ctx->layers.end())
        return fail(DKV_ERR_NOT_REGISTERED, "dkv_extend_ragged: layer %d not registered - call dkv_layer_register first",
                    layer_id);
    const LayerState& L = it->second;
    DKV_REQUIRE(Q && O && s_new_host && past_host && rows_host, "NULL argument");
    DKV_REQUIRE(B > 0 && nh_q > 0 && nh_q % L.d.nh_kv == 0, "bad sizes");
    const bool project = (X != nullptr), paged = (page_table != nullptr);
    if (project) DKV_REQUIRE(L.has_weights, "layer %d has no projection weights registered", layer_id);
    DKV_REQUIRE(!(project && paged), "projection into a paged pool is not supported: store the rows, then pass X = NULL");
    if (paged) DKV_REQUIRE(pt_stride > 0, "pt_stride must be positive with a page table");
    else DKV_REQUIRE(L.d.row_stride > 0, "layer %d was registered without row_stride and no page table was given", layer_id);
    const int nh_kv = L.d.nh_kv;
    const int g_total = nh_q / nh_kv;
    int G = 1;
    while (G < 128 && g_total % (2 * G) == 0) G *= 2;
    const int nsub = g_total / G, TQ = kExtTile / G;

    long long T = 0, kv_total = 0, n_items = 0;
    for (int b = 0; b < B; ++b) {
        DKV_REQUIRE(s_new_host[b] > 0 && past_host[b] >= 0 && rows_host[b] >= 0, "request %d: bad lengths or row", b);
        const long long tot = static_cast<long long>(past_host[b]) + s_new_host[b];
        if (paged) DKV_REQUIRE(((tot - 1) >> L.page_shift) < pt_stride, "request %d does not fit a page-table row", b);
        else DKV_REQUIRE(tot <= L.d.row_stride, "request %d: seqlen_past + S_new (%lld) exceeds the pool row (%lld)", b, tot,
                         (long long)L.d.row_stride);
        T += s_new_host[b];
        kv_total += tot;
        n_items += (s_new_host[b] + 2 * TQ - 1) / (2 * TQ);
    }
    DKV_REQUIRE(T < (1ll << 30) && kv_total < (1ll << 30), "batch too large");
    const bool stage = paged || L.pool_on_host;
    DKV_CUDA(cudaSetDevice(ctx->device));
    cudaStream_t st = static_cast<cudaStream_t>(stream);

    // ---- metadata: [s_new | past | q_row0 | slot0 | rows | kv_off (B + 1) | pad | items (2 per entry, 8-byte aligned)] ----
    const size_t items_at = static_cast<size_t>(6) * B + 2;
    const size_t ints = items_at + 2 * static_cast<size_t>(n_items);
    int rc = ensure_ragged(ctx, ints);
    if (rc != DKV_OK) return rc;
    if (ctx->ragged_pending) {           // the previous upload must have left the host mirror
        DKV_CUDA(cudaEventSynchronize(ctx->ev_ragged));
        ctx->ragged_pending = false;
    }
    int* hs_new = ctx->ragged_host;
    int* hpast = hs_new + B;
    int* hq0 = hpast + B;
    int* hslot0 = hq0 + B;
    int* hrows = hslot0 + B;
    int* hkvoff = hrows + B;
    int* hitems = ctx->ragged_host + items_at;
    struct Item { long long key; int b, qt; };
    std::vector<Item> items;
    items.reserve(static_cast<size_t>(n_items));
    int q_acc = 0, kv_acc = 0;
    for (int b = 0; b < B; ++b) {
        hs_new[b] = s_new_host[b];
        hpast[b] = past_host[b];
        hq0[b] = q_acc;
        hrows[b] = rows_host[b];
        hkvoff[b] = kv_acc;
        hslot0[b] = stage ? kv_acc : static_cast<int>(static_cast<long long>(rows_host[b]) * L.d.row_stride);
        const int n_qt = (s_new_host[b] + 2 * TQ - 1) / (2 * TQ);
        for (int qt = 0; qt < n_qt; ++qt) {
            long long end = is_causal ? static_cast<long long>(past_host[b]) + static_cast<long long>(qt + 1) * 2 * TQ
                                      : static_cast<long long>(past_host[b]) + s_new_host[b];
            items.push_back({end, b, qt});
        }
        q_acc += s_new_host[b];
        kv_acc += past_host[b] + s_new_host[b];
    }
    hkvoff[B] = kv_acc;
    std::stable_sort(items.begin(), items.end(), [](const Item& a, const Item& c) { return a.key > c.key; });   // longest first
    for (size_t i = 0; i < items.size(); ++i) {
        hitems[2 * i] = items[i].b;
        hitems[2 * i + 1] = items[i].qt;
    }
    DKV_CUDA(cudaMemcpyAsync(ctx->ragged_dev, ctx->ragged_host, ints * sizeof(int), cudaMemcpyHostToDevice, st));
    DKV_CUDA(cudaEventRecord(ctx->ev_ragged, st));
    ctx->ragged_pending = true;
    const int* ds_new = ctx->ragged_dev;
    const int* dpast = ds_new + B;
    const int* dq0 = dpast + B;
    const int* dslot0 = dq0 + B;
    const int* drows = dslot0 + B;
    const int* dkvoff = drows + B;
    const int2* ditems = reinterpret_cast<const int2*>(ctx->ragged_dev + items_at);

    const size_t stage_bytes = stage ? static_cast<size_t>(kv_total) * nh_kv * 256 : 0;
    ScratchPlan sp = plan_scratch(ctx, T, nh_q, nh_kv, L.d.hidden, project, false, stage_bytes);
    rc = ensure_scratch(ctx, sp, st);
    if (rc != DKV_OK) return rc;
    uint8_t* base = ctx->scratch.ptr;
    uint4* ks = stage ? reinterpret_cast<uint4*>(ctx->stage.ptr + sp.stage_k) : nullptr;
    uint4* vs = stage ? reinterpret_cast<uint4*>(ctx->stage.ptr + sp.stage_v) : nullptr;
    // Host pool with projection: the new rows are projected straight into the staging copy, which the attention
    // reads, and go to the host pool from there on the side stream while the attention runs - they cross the host
    // link once, outside the critical path, instead of twice inside it.
    const bool proj_to_stage = project && stage;
    void* k_host = L.pool_on_host ? const_cast<void*>(static_cast<const void*>(L.d.k_pool)) : nullptr;   // host address of the pinned pool
    void* v_host = L.pool_on_host ? const_cast<void*>(static_cast<const void*>(L.d.v_pool)) : nullptr;
    if (project) {
        int* tok_pos = reinterpret_cast<int*>(base + sp.tok_pos);
        int* tok_slot = reinterpret_cast<int*>(base + sp.tok_slot);
        int* tok_pool_slot = reinterpret_cast<int*>(base + sp.vseq);
        extend_prep_ragged_kernel<<<static_cast<int>((T + 255) / 256), 256, 0, st>>>(
            B, static_cast<int>(T), dq0, dpast, drows, L.d.row_stride, proj_to_stage ? dkvoff : nullptr, tok_pos, tok_slot,
            tok_pool_slot);
        DKV_CUDA(cudaGetLastError());
        ctx->launches += 1;
        rc = launch_projection(ctx, L, X, static_cast<int>(T), tok_pos, tok_slot, true, nullptr,
                               reinterpret_cast<float*>(base + sp.splitk), st, false, proj_to_stage ? ks : nullptr,
                               proj_to_stage ? vs : nullptr, kv_total);
        if (rc != DKV_OK) return rc;
        if (proj_to_stage) {
            DKV_CUDA(cudaEventRecord(ctx->ev_fork, st));
            DKV_CUDA(cudaStreamWaitEvent(ctx->side, ctx->ev_fork, 0));
            // Contiguous rows: one copy-engine transfer per request and tensor (the faster way over the host link).
            const size_t row_bytes = static_cast<size_t>(nh_kv) * 256;
            for (int b = 0; b < B; ++b) {
                const size_t src = (static_cast<size_t>(hkvoff[b]) + past_host[b]) * row_bytes;
                const size_t dst = (static_cast<size_t>(rows_host[b]) * L.d.row_stride + past_host[b]) * row_bytes;
                const size_t bytes = static_cast<size_t>(s_new_host[b]) * row_bytes;
                DKV_CUDA(cudaMemcpyAsync(static_cast<uint8_t*>(k_host) + dst, reinterpret_cast<uint8_t*>(ks) + src, bytes,
                                         cudaMemcpyDeviceToHost, ctx->side));
                DKV_CUDA(cudaMemcpyAsync(static_cast<uint8_t*>(v_host) + dst, reinterpret_cast<uint8_t*>(vs) + src, bytes,
                                         cudaMemcpyDeviceToHost, ctx->side));
            }
            DKV_CUDA(cudaEventRecord(ctx->ev_join, ctx->side));
        }
    }
    CUtensorMap tmQ, tmKs, tmVs;
    rc = encode_tile_map(&tmQ, Q, T, nh_q, G, TQ);
    if (rc != DKV_OK) return rc;
    const CUtensorMap* tmK = &L.tmK_128;
    const CUtensorMap* tmV = &L.tmV_128;
    if (stage && !paged && k_host != nullptr) {
        // Contiguous rows of a host pool: the copy engines bring them in (55.6 against 51.5 GB/s for SM reads).
        const size_t row_bytes = static_cast<size_t>(nh_kv) * 256;
        for (int b = 0; b < B; ++b) {
            const int n = proj_to_stage ? past_host[b] : past_host[b] + s_new_host[b];
            if (n == 0) continue;
            const size_t src = static_cast<size_t>(rows_host[b]) * L.d.row_stride * row_bytes;
            const size_t dst = static_cast<size_t>(hkvoff[b]) * row_bytes;
            DKV_CUDA(cudaMemcpyAsync(reinterpret_cast<uint8_t*>(ks) + dst, static_cast<const uint8_t*>(k_host) + src,
                                     static_cast<size_t>(n) * row_bytes, cudaMemcpyHostToDevice, st));
            DKV_CUDA(cudaMemcpyAsync(reinterpret_cast<uint8_t*>(vs) + dst, static_cast<const uint8_t*>(v_host) + src,
                                     static_cast<size_t>(n) * row_bytes, cudaMemcpyHostToDevice, st));
        }
    } else if (stage) {
        stage_rows_ragged_kernel<<<ctx->sm_count * 8, 256, 0, st>>>(ks, vs, static_cast<const uint4*>(L.k_dev),
                                                                    static_cast<const uint4*>(L.v_dev), B, dkvoff, drows,
                                                                    L.d.row_stride, nh_kv * 16, page_table, pt_stride,
                                                                    L.page_shift, proj_to_stage ? dpast : nullptr);
        DKV_CUDA(cudaGetLastError());
        ctx->launches += 1;
    }
    if (stage) {                     // the attention reads the staging copy
        if ((rc = encode_tile_map(&tmKs, ks, kv_total, nh_kv, 1, kExtTile)) != DKV_OK) return rc;
        if ((rc = encode_tile_map(&tmVs, vs, kv_total, nh_kv, 1, kExtTile)) != DKV_OK) return rc;
        tmK = &tmKs;
        tmV = &tmVs;
    }
    ExtendParams ep{};
    ep.nh_q = nh_q;
    ep.nh_kv = nh_kv;
    ep.G = G;
    ep.g_total = g_total;
    ep.nsub = nsub;
    ep.is_causal = is_causal;
    ep.scale_log2 = softmax_scale * 1.4426950408889634f;
    ep.out = static_cast<__nv_bfloat16*>(O);
    ep.status = ctx->status;
    ep.items = ditems;
    ep.r_s_new = ds_new;
    ep.r_past = dpast;
    ep.r_q_row0 = dq0;
    ep.r_slot0 = dslot0;
    dim3 grid(nh_kv * nsub, static_cast<unsigned>(n_items), 1);
    extend_attn_pp_kernel<<<grid, kPpThreads, kPpSmem, st>>>(tmQ, *tmK, *tmV, ep);
    DKV_CUDA(cudaGetLastError());
    ctx->launches += 1;
    if (proj_to_stage) DKV_CUDA(cudaStreamWaitEvent(st, ctx->ev_join, 0));   // the pool holds the new rows when the call's work is done
    return DKV_OK;
}

int dkv_scatter_kv(dkv_context* ctx, void* k_pool, void* v_pool, int64_t n_slots, int64_t k_row_bytes,
                   int64_t v_row_bytes, const void* loc, int loc_is_int64, const void* cache_k, const void* cache_v,
                   int64_t n_tokens, void* stream) {
    DKV_REQUIRE(ctx != nullptr && k_pool && v_pool && loc && cache_k && cache_v, "NULL argument");
    DKV_REQUIRE(n_slots > 0 && n_tokens >= 0, "bad sizes");
    DKV_REQUIRE(k_row_bytes > 0 && k_row_bytes % 16 == 0 && v_row_bytes > 0 && v_row_bytes % 16 == 0,
                "token rows must be multiples of 16 bytes");
    if (n_tokens == 0) return DKV_OK;
    DKV_CUDA(cudaSetDevice(ctx->device));
    void *kd = nullptr, *vd = nullptr;
    int rc = device_pointer_of(k_pool, &kd, "k_pool");
    if (rc != DKV_OK) return rc;
    if ((rc = device_pointer_of(v_pool, &vd, "v_pool")) != DKV_OK) return rc;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int grid = static_cast<int>(n_tokens);
    if (loc_is_int64) {
        scatter_rows_kernel<long long><<<grid, 128, 0, st>>>(static_cast<uint4*>(kd), static_cast<const uint4*>(cache_k),
                                                            static_cast<const long long*>(loc), n_slots,
                                                            static_cast<int>(k_row_bytes / 16), ctx->status);
        scatter_rows_kernel<long long><<<grid, 128, 0, st>>>(static_cast<uint4*>(vd), static_cast<const uint4*>(cache_v),
                                                            static_cast<const long long*>(loc), n_slots,
                                                            static_cast<int>(v_row_bytes / 16), ctx->status);
    } else {
        scatter_rows_kernel<int><<<grid, 128, 0, st>>>(static_cast<uint4*>(kd), static_cast<const uint4*>(cache_k),
                                                      static_cast<const int*>(loc), n_slots,
                                                      static_cast<int>(k_row_bytes / 16), ctx->status);
        scatter_rows_kernel<int><<<grid, 128, 0, st>>>(static_cast<uint4*>(vd), static_cast<const uint4*>(cache_v),
                                                      static_cast<const int*>(loc), n_slots,
                                                      static_cast<int>(v_row_bytes / 16), ctx->status);
    }
    DKV_CUDA(cudaGetLastError());
    return DKV_OK;
}

int dkv_stream_copy(dkv_context* ctx, void* dst, const void* src, int64_t bytes, void* stream) {
    DKV_REQUIRE(ctx != nullptr && dst != nullptr && src != nullptr, "NULL argument");
    DKV_REQUIRE(bytes > 0 && bytes % 16 == 0, "bytes must be a positive multiple of 16");
    DKV_CUDA(cudaSetDevice(ctx->device));
    void* src_dev = nullptr;
    int rc = device_pointer_of(const_cast<void*>(src), &src_dev, "src");
    if (rc != DKV_OK) return rc;
    stream_copy_kernel<<<ctx->sm_count * 8, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<uint4*>(dst), static_cast<const uint4*>(src_dev), bytes / 16);
    DKV_CUDA(cudaGetLastError());
    return DKV_OK;
}

}  // extern "C"
