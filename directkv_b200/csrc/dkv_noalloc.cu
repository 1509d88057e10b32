// dkv_decode_noalloc: decode attention for callers that must not allocate device memory.
//
// Who needs this: code that runs while a CUDA graph is being captured or inside a serving loop
// whose memory plan is frozen (every byte of HBM was handed to a KV-cache allocator at start-up),
// and plugins loaded into a host process that forbids cudaMalloc / cudaFree from extension code
// because those calls synchronise the device or fragment its pool.  The regular entry points keep
// their scratch in a context that grows with cudaMalloc; this one keeps it in the fixed
// file-scope array below, so it needs no context and allocates nothing - no cudaMalloc, no
// cudaFree, no allocating library routine.
//
// The price: a fixed ceiling (kScratchBytes, held by every GPU that loads the library until the
// process exits) and one scratch shared by all calls.  Calls that overlap on the GPU (different
// streams, or different host threads on one device) race on it; issue them on one stream, or
// order them with events.
#include "../../include/directkv_b200.h"

#include <cstdarg>
#include <cstdio>
#include <mutex>

// This translation unit gets its own copy of the kernels, in a namespace of its own, so that it
// links beside dkv_capi.cu (which instantiates the same header) without touching that file.
#define dkv dkv_noalloc_impl
#include "dkv_attn.cuh"
#undef dkv

namespace {

using namespace dkv_noalloc_impl;

// ---- the scratch ------------------------------------------------------------------------------
// Layout: [0, 256) status word | [256, kPartialsOffset) cum_tiles | [kPartialsOffset, end) partials.
constexpr size_t kScratchBytes = 4u << 20;      // 4 MiB per GPU
constexpr size_t kCumOffset = 256;
constexpr size_t kPartialsOffset = 8192;
constexpr int kMaxBatch = static_cast<int>((kPartialsOffset - kCumOffset) / 4) - 1;   // 1983 requests

static __device__ __align__(256) unsigned char g_noalloc_scratch[kScratchBytes];

// In host code `g_noalloc_scratch` is only a handle for the runtime, never a device address:
// the address each device gave the array is looked up once per device and cached here.
constexpr int kMaxDevices = 64;
unsigned char* g_scratch_dev[kMaxDevices] = {nullptr};
int g_sm_count[kMaxDevices] = {0};
std::mutex g_setup_mutex;

// Error text goes to the caller's buffer (dkv_noalloc_args.err_buf): this file keeps no state of
// its own besides the scratch address table.
thread_local char* t_err_buf = nullptr;
thread_local int t_err_len = 0;

int fail(int code, const char* fmt, ...) {
    if (t_err_buf != nullptr && t_err_len > 0) {
        va_list ap;
        va_start(ap, fmt);
        vsnprintf(t_err_buf, static_cast<size_t>(t_err_len), fmt, ap);
        va_end(ap);
    }
    return code;
}

#define NA_CUDA(expr)                                                                                      \
    do {                                                                                                   \
        cudaError_t _e = (expr);                                                                           \
        if (_e != cudaSuccess)                                                                             \
            return fail(DKV_ERR_CUDA, "%s failed: %s (%s:%d)", #expr, cudaGetErrorString(_e), __FILE__, __LINE__); \
    } while (0)

#define NA_REQUIRE(cond, ...)                                   \
    do {                                                        \
        if (!(cond)) return fail(DKV_ERR_INVALID, __VA_ARGS__); \
    } while (0)

constexpr int kWarpsG12 = 16, kStagesG12 = 1;   // streaming-kernel shape for 1 or 2 query heads per KV head
constexpr int kWarpsG4 = 8, kStagesG4 = 3;      // and for 4

template <int G, int NW, int NST>
constexpr size_t smem_bytes() {
    return attn_dyn_smem_bytes<NW, NST>();
}

// Once per device, with that device current: find the array's address on this device and raise
// the kernels' dynamic shared-memory limit.  Neither call allocates.
int setup_device(int dev) {
    std::lock_guard<std::mutex> lock(g_setup_mutex);
    if (g_scratch_dev[dev] != nullptr) return DKV_OK;
    cudaDeviceProp prop;
    NA_CUDA(cudaGetDeviceProperties(&prop, dev));
    if (prop.major != 10)
        return fail(DKV_ERR_UNSUPPORTED, "device %d is sm_%d%d; this library is built for sm_100a only", dev, prop.major,
                    prop.minor);
    unsigned char* ptr = nullptr;
    NA_CUDA(cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_noalloc_scratch));
    NA_CUDA(cudaFuncSetAttribute(attn_partial_kernel<1, kWarpsG12, kStagesG12>,
                                 cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 static_cast<int>(smem_bytes<1, kWarpsG12, kStagesG12>())));
    NA_CUDA(cudaFuncSetAttribute(attn_partial_kernel<2, kWarpsG12, kStagesG12>,
                                 cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 static_cast<int>(smem_bytes<2, kWarpsG12, kStagesG12>())));
    NA_CUDA(cudaFuncSetAttribute(attn_partial_kernel<4, kWarpsG4, kStagesG4>,
                                 cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 static_cast<int>(smem_bytes<4, kWarpsG4, kStagesG4>())));
    g_sm_count[dev] = prop.multiProcessorCount;
    g_scratch_dev[dev] = ptr;
    return DKV_OK;
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// Fills a caller-provided descriptor on the host; the pool itself is not touched.
int encode_pool(CUtensorMap* m, void* base, int64_t n_slots, int nh, int rows) {
    static EncodeTiledFn g_encode = nullptr;      // looked up once, under the same lock as the rest of the set-up
    EncodeTiledFn fn = nullptr;
    {
        std::lock_guard<std::mutex> lock(g_setup_mutex);
        if (!g_encode) {
            void* p = nullptr;
            cudaDriverEntryPointQueryResult q;
            if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
                q != cudaDriverEntryPointSuccess)
                return fail(DKV_ERR_CUDA, "cuTensorMapEncodeTiled entry point not available");
            g_encode = reinterpret_cast<EncodeTiledFn>(p);
        }
        fn = g_encode;
    }
    cuuint64_t gdim[3] = {128, (cuuint64_t)nh, (cuuint64_t)n_slots};
    cuuint64_t gstr[2] = {256, (cuuint64_t)nh * 256};
    cuuint32_t box[3] = {128, 1, (cuuint32_t)rows};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, base, gdim, gstr, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(DKV_ERR_CUDA, "cuTensorMapEncodeTiled failed: %d", (int)r);
    return DKV_OK;
}

// Address under which the current device reaches `p`: device memory of THIS device, or page-locked host memory.
// Memory of another GPU is refused: the kernels would read it over NVLink, or fault where there is no peer access.
int device_address(const void* p, int dev, bool allow_host, void** out, const char* what) {
    cudaPointerAttributes attr;
    NA_CUDA(cudaPointerGetAttributes(&attr, p));
    if (attr.type == cudaMemoryTypeDevice || attr.type == cudaMemoryTypeManaged) {
        if (attr.type == cudaMemoryTypeDevice && attr.device != dev)
            return fail(DKV_ERR_INVALID, "%s lives on device %d but the current device is %d", what, attr.device, dev);
        *out = const_cast<void*>(p);
        return DKV_OK;
    }
    if (!allow_host) return fail(DKV_ERR_INVALID, "%s must be device memory of the current device", what);
    if (attr.type == cudaMemoryTypeHost && attr.devicePointer != nullptr) {
        *out = attr.devicePointer;
        return DKV_OK;
    }
    return fail(DKV_ERR_INVALID, "%s must be pinned (page-locked) host memory or device memory", what);
}

}  // namespace

extern "C" int dkv_decode_noalloc(const dkv_noalloc_args* a, void* stream) {
    t_err_buf = nullptr;
    t_err_len = 0;
    if (a == nullptr) return DKV_ERR_INVALID;
    t_err_buf = a->err_buf;
    t_err_len = a->err_buf_len;
    if (t_err_buf != nullptr && t_err_len > 0) t_err_buf[0] = 0;
    NA_REQUIRE(a->k_pool && a->v_pool && a->q && a->out && a->seq_lens && a->page_table, "NULL tensor pointer");
    NA_REQUIRE(a->batch > 0 && a->nh_kv > 0 && a->nh_q > 0 && a->nh_q % a->nh_kv == 0,
               "batch, nh_kv, nh_q must be positive and nh_q a multiple of nh_kv");
    NA_REQUIRE(a->n_slots > 0 && a->pt_stride > 0, "n_slots and pt_stride must be positive");
    NA_REQUIRE(a->n_slots <= static_cast<int64_t>(INT32_MAX), "n_slots (%lld) exceeds the 2^31 - 1 slots a pool can address",
               (long long)a->n_slots);
    NA_REQUIRE(a->page_size >= 1 && (a->page_size & (a->page_size - 1)) == 0, "page_size (%d) must be a power of two",
               a->page_size);
    NA_REQUIRE(a->q_stride >= static_cast<int64_t>(a->nh_q) * 128 && a->q_stride % 8 == 0 &&
                   a->out_stride >= static_cast<int64_t>(a->nh_q) * 128 && a->out_stride % 4 == 0,
               "q_stride / out_stride too small or unaligned");
    NA_REQUIRE((reinterpret_cast<uintptr_t>(a->q) & 15) == 0 && (reinterpret_cast<uintptr_t>(a->out) & 7) == 0 &&
                   (reinterpret_cast<uintptr_t>(a->k_pool) & 15) == 0 && (reinterpret_cast<uintptr_t>(a->v_pool) & 15) == 0,
               "q / out / pools are not aligned");
    int dev = 0;
    NA_CUDA(cudaGetDevice(&dev));
    NA_REQUIRE(dev >= 0 && dev < kMaxDevices, "device index %d out of range", dev);
    int rc = setup_device(dev);   // first call on this device: do it before any stream capture
    if (rc != DKV_OK) return rc;

    // ---- does it fit in the built-in scratch? ----------------------------------------------------
    const int g_total = a->nh_q / a->nh_kv;
    const int G = (g_total % 4 == 0) ? 4 : (g_total % 2 == 0) ? 2 : 1;
    const int nsub = g_total / G;
    const int warps = (G == 4) ? kWarpsG4 : kWarpsG12;
    const int ctas = g_sm_count[dev];
    const size_t records = static_cast<size_t>(ctas) * warps + static_cast<size_t>(a->batch) * a->nh_kv * nsub;
    const size_t need = records * G * kPartialStride * sizeof(float);
    if (a->batch > kMaxBatch)
        return fail(DKV_ERR_UNSUPPORTED, "dkv_decode_noalloc: batch %d exceeds the built-in limit of %d requests",
                    a->batch, kMaxBatch);
    if (need > kScratchBytes - kPartialsOffset)
        return fail(DKV_ERR_UNSUPPORTED,
                    "dkv_decode_noalloc: batch %d x %d KV heads x %d query heads needs %zu bytes of partials but the "
                    "built-in scratch holds %zu; use dkv_decode (which allocates) for this size",
                    a->batch, a->nh_kv, a->nh_q, need, kScratchBytes - kPartialsOffset);

    void *kd = nullptr, *vd = nullptr, *unused = nullptr;
    if ((rc = device_address(a->k_pool, dev, true, &kd, "k_pool")) != DKV_OK) return rc;
    if ((rc = device_address(a->v_pool, dev, true, &vd, "v_pool")) != DKV_OK) return rc;
    if ((rc = device_address(a->q, dev, false, &unused, "q")) != DKV_OK) return rc;
    if ((rc = device_address(a->out, dev, false, &unused, "out")) != DKV_OK) return rc;
    if (a->status_out != nullptr && (rc = device_address(a->status_out, dev, false, &unused, "status_out")) != DKV_OK) return rc;
    const int rows_per_box = a->page_size < kTileTokens ? a->page_size : kTileTokens;
    CUtensorMap tmK, tmV;
    if ((rc = encode_pool(&tmK, kd, a->n_slots, a->nh_kv, rows_per_box)) != DKV_OK) return rc;
    if ((rc = encode_pool(&tmV, vd, a->n_slots, a->nh_kv, rows_per_box)) != DKV_OK) return rc;

    cudaStream_t st = static_cast<cudaStream_t>(stream);
    unsigned char* base = g_scratch_dev[dev];
    unsigned int* status = reinterpret_cast<unsigned int*>(base);
    int* cum = reinterpret_cast<int*>(base + kCumOffset);
    float* partials = reinterpret_cast<float*>(base + kPartialsOffset);
    // The array keeps whatever the previous call left.  cum_tiles and every partial record that is read are
    // rewritten by this call's own kernels.  The status word: a caller that passes status_out owns the word the
    // kernels OR their failure bits into (it clears and reads it when it likes - the way to see a device-side
    // failure without a synchronising call, e.g. for a call recorded into a graph); otherwise the word inside
    // the array is used and cleared here, stream-ordered, so that sync_and_check reports this call only.
    if (a->status_out != nullptr) status = a->status_out;
    else NA_CUDA(cudaMemsetAsync(status, 0, sizeof(unsigned int), st));

    PrepParams prep{};
    prep.seq_lens = a->seq_lens;
    prep.batch = a->batch;
    prep.n_new = 0;
    prep.cum_tiles = cum;
    attn_prep_kernel<<<1, 256, 0, st>>>(prep);
    NA_CUDA(cudaGetLastError());

    AttnParams ap{};
    ap.q = static_cast<const __nv_bfloat16*>(a->q);
    ap.q_stride = a->q_stride;
    ap.page_table = a->page_table;
    ap.row_map = nullptr;
    ap.seq_lens = a->seq_lens;
    ap.cum_tiles = cum;
    ap.partials = partials;
    ap.status = status;
    ap.batch = a->batch;
    ap.nh_q = a->nh_q;
    ap.nh_kv = a->nh_kv;
    ap.g_total = g_total;
    ap.nsub = nsub;
    ap.pt_stride = a->pt_stride;
    ap.pt_rows = a->batch;
    ap.page_size = a->page_size;
    ap.page_shift = 0;
    while ((1 << ap.page_shift) < a->page_size) ++ap.page_shift;
    ap.rows_per_box = rows_per_box;
    ap.row_stride = 0;
    ap.n_new = 0;
    ap.total_warps = ctas * warps;
    ap.min_units = 1;
    ap.scale_log2 = a->softmax_scale * 1.4426950408889634f;

    if (G == 4)
        attn_partial_kernel<4, kWarpsG4, kStagesG4><<<ctas, kWarpsG4 * 32, smem_bytes<4, kWarpsG4, kStagesG4>(), st>>>(tmK, tmV, ap);
    else if (G == 2)
        attn_partial_kernel<2, kWarpsG12, kStagesG12><<<ctas, kWarpsG12 * 32, smem_bytes<2, kWarpsG12, kStagesG12>(), st>>>(tmK, tmV, ap);
    else
        attn_partial_kernel<1, kWarpsG12, kStagesG12><<<ctas, kWarpsG12 * 32, smem_bytes<1, kWarpsG12, kStagesG12>(), st>>>(tmK, tmV, ap);
    NA_CUDA(cudaGetLastError());

    MergeParams mp{};
    mp.a = ap;
    mp.G = G;
    mp.kv_new = nullptr;
    mp.out = static_cast<__nv_bfloat16*>(a->out);
    mp.out_stride = a->out_stride;
    mp.lse = a->lse_out;
    mp.part_out = nullptr;
    const long long rows = static_cast<long long>(a->batch) * a->nh_q;
    if (static_cast<long long>(a->batch) * a->nh_kv * nsub * 8 < ap.total_warps)
        attn_merge_kernel<8><<<static_cast<int>(rows), kMergeThreads, 0, st>>>(mp);
    else
        attn_merge_kernel<1><<<static_cast<int>((rows + 7) / 8), kMergeThreads, 0, st>>>(mp);
    NA_CUDA(cudaGetLastError());

    if (a->sync_and_check) {
        unsigned int h = 0;
        NA_CUDA(cudaStreamSynchronize(st));
        NA_CUDA(cudaMemcpy(&h, status, sizeof(h), cudaMemcpyDeviceToHost));
        if (h != 0)
            return fail(DKV_ERR_DEVICE_STATUS, "dkv_decode_noalloc: device status 0x%x (bit 0: a bounded wait ran out; "
                        "bit 5: a length or row led outside the page table)", h);
    }
    return DKV_OK;
}
