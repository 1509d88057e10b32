// K/V projection of one or two new tokens (the decode step of one or two requests) as a stream over the weight rows
// on the CUDA cores.
//
// With so few tokens the product  K_h(t, d) = sum_k Wk_h(d, k) X(t, k)  is a matrix-vector product: every weight
// is used once per token, nothing is gained from the tensor cores, and what the tensor-core kernel pays around
// its stream (tensor-memory allocation, a 16-token operand tile, fp32 slices through global memory for the
// split of the hidden dimension, a last-arriver pass) is most of a short step.  Here every WARP works alone on
// one pair of weight rows at a time - dimensions j and j + 64 of one head's K (the two that the Neox rotation
// mixes) or V: no barrier of the CTA and no exchange between warps inside the loop.  The pair arrives in two
// (or four) column segments, each by one bulk copy per row, into the warp's own two-stage ring: while one
// segment is multiplied the next is on its way, and as soon as a segment has been read its slot takes the same
// segment of the warp's next pair.  (Copies of 2 KB are bound by the rate at which an SM's copy unit takes
// requests - about 2.5 TB/s over the GPU - so the segments are as long as the shared memory allows.)  The
// tokens' activations stay in shared memory for the whole kernel; a lane multiplies 8 columns per step and token
// in fp32 and unpacks the activations once for both rows.
//
// Same contract as proj_rope_decode_kernel (ProjParams): round to bf16, rotate K at the token's absolute
// position, round again, store to the pool and to kv_new (csrc/directKV_kernel.cuh:430-546 in the reference).
// 128 threads, under 96 registers and at most 96 KB of shared memory: the CTA fits beside a streaming CTA.
#pragma once

#include "dkv_proj.cuh"

namespace dkv {

constexpr int kGvMaxTokens = 2;                      // with more tokens the tensor-core kernel is the faster one again
constexpr int kGvWarps = 4;
constexpr int kGvStages = 2;                         // segments in flight per warp
constexpr int kGvCtrlBytes = 4096;                   // barriers [4][2], cos | sin rows [2][128]
constexpr int kGvSmemBudget = 96 * 1024;

__host__ __device__ constexpr int gv_x_bytes(int T, int H) { return T * H * 2; }
// Column segments a row pair is cut into: two if the rings fit beside the activations, else four.
__host__ __device__ constexpr int gv_segments(int T, int H) {
    return gv_x_bytes(T, H) + kGvCtrlBytes + kGvWarps * kGvStages * (2 * (H / 2) * 2) <= kGvSmemBudget ? 2 : 4;
}
__host__ __device__ constexpr int gv_stage_bytes(int T, int H) { return 2 * (H / gv_segments(T, H)) * 2; }   // both rows
__host__ __device__ constexpr size_t gv_smem_bytes(int T, int H) {
    return static_cast<size_t>(gv_x_bytes(T, H)) + static_cast<size_t>(kGvWarps) * kGvStages * gv_stage_bytes(T, H) + kGvCtrlBytes;
}
// Whether the kernel takes this shape: segments in whole 256-column steps, and everything within the budget.
__host__ __device__ constexpr bool gv_supports(int T, int H) {
    return T >= 1 && T <= kGvMaxTokens && H > 0 && H % 1024 == 0 && gv_smem_bytes(T, H) <= static_cast<size_t>(kGvSmemBudget);
}
static_assert(gv_supports(1, 4096) && gv_segments(2, 4096) == 2 && gv_supports(2, 7168) && gv_segments(2, 7168) == 4 &&
              gv_supports(1, 8192) && !gv_supports(2, 8192) && !gv_supports(3, 4096), "ring sizes");

// Bulk copy global -> this CTA's shared memory, completion counted in bytes on an mbarrier (no multicast).
__device__ __forceinline__ void bulk_load(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     smem_u32(smem_dst)),
                 "l"(reinterpret_cast<uint64_t>(gsrc)), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}

__device__ __forceinline__ float bf16_lo(uint32_t u) { return __uint_as_float(u << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t u) { return __uint_as_float(u & 0xffff0000u); }

// grid: up to one CTA per SM; warp gw = blockIdx.x * 4 + warp takes the row pairs u = gw, gw + 4 * gridDim.x, ...
// of nh_kv * 128 (u = h * 128 + kv * 64 + j).  x is [T, H] bf16, wk / wv are [nh_kv, 128, H] bf16.
template <int T>
__global__ void __launch_bounds__(128, 5)   // at most 96 registers: the CTA must fit beside a streaming CTA
proj_rope_gemv_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ wk,
                      const __nv_bfloat16* __restrict__ wv, const ProjParams p) {
    extern __shared__ __align__(128) uint8_t gv_smem[];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int H = p.H;
    const int n_seg = gv_segments(T, H);
    const int seg_cols = H / n_seg;
    const int seg_bytes = seg_cols * 2;                    // of one row
    const int stage_bytes = 2 * seg_bytes;
    uint8_t* xs = gv_smem;                                                               // [T][H] bf16
    uint8_t* ring = gv_smem + gv_x_bytes(T, H) + warp * kGvStages * stage_bytes;         // this warp's two stages
    uint8_t* ctrl = gv_smem + gv_x_bytes(T, H) + kGvWarps * kGvStages * stage_bytes;
    uint64_t* full = reinterpret_cast<uint64_t*>(ctrl) + warp * kGvStages;                // [4][2]
    float* cs_s = reinterpret_cast<float*>(ctrl + 1024);                                  // [T][128]: cos | sin at each token's position

    const int n_units = p.nh_kv * 128;
    const int gw = static_cast<int>(blockIdx.x) * kGvWarps + warp, n_gw = static_cast<int>(gridDim.x) * kGvWarps;
    const int my_units = gw < n_units ? (n_units - gw + n_gw - 1) / n_gw : 0;
    const int total = my_units * n_seg;                    // this warp's stages over the whole kernel

    // Stage f of this warp's sequence: segment f % n_seg of both rows of pair gw + (f / n_seg) * n_gw.
    auto issue = [&](int f) {
        const int u = gw + (f / n_seg) * n_gw;
        const int h = u >> 7, kv = (u >> 6) & 1, j = u & 63;
        const __nv_bfloat16* row = (kv ? wv : wk) + (static_cast<size_t>(h) * 128 + j) * H + (f % n_seg) * seg_cols;
        const int s = f % kGvStages;
        uint8_t* dst = ring + s * stage_bytes;
        mbar_arrive_expect_tx(&full[s], static_cast<uint32_t>(stage_bytes));
        bulk_load(dst, row, static_cast<uint32_t>(seg_bytes), &full[s]);
        bulk_load(dst + seg_bytes, row + static_cast<size_t>(64) * H, static_cast<uint32_t>(seg_bytes), &full[s]);
    };
    int issued = 0;
    if (lane == 0) {
        for (int s = 0; s < kGvStages; ++s) mbar_init(&full[s], 1);
        fence_mbar_init();
        fence_proxy_async_smem();
        for (; issued < total && issued < kGvStages; ++issued) issue(issued);
    }
    __syncwarp();

    // What depends on the token only is fetched once, while the first weight segments are on their way: the row of
    // the rotation table at the token's position, and (lane t, which finishes token t) its pool slot.  Inside the
    // loop over the row pairs nothing waits for global memory any more.
    const bool rotate = p.cos_sin != nullptr && proj_has_pos(p);
    if (rotate) {
        for (int idx = tid; idx < T * kProjHead; idx += 128) {
            const int pos = proj_tok_pos(p, idx >> 7);
            const bool in_table = pos >= 0 && pos < p.max_pos;
            // out of the table: no rotation (cos 1, sin 0) and the status bit, as in the other projection kernels
            cs_s[idx] = in_table ? __ldg(p.cos_sin + static_cast<size_t>(pos) * kProjHead + (idx & 127)) : ((idx & 127) < 64 ? 1.f : 0.f);
            if (!in_table && (idx & 127) == 0 && blockIdx.x == 0) atomicOr(p.status, kStatusBadPosition);
        }
    }
    long long my_slot = -1;
    if (lane < T) my_slot = proj_tok_slot(p, lane);
    // The tokens' activations.
    for (int idx = tid; idx < T * H / 8; idx += 128)
        reinterpret_cast<uint4*>(xs)[idx] = __ldg(reinterpret_cast<const uint4*>(x) + idx);
    __syncthreads();                                       // the only barrier of the CTA

    const int steps = seg_cols / 256;                      // 256-column steps per segment
    bool ok = true;
    int f = 0, consumed = 0;                               // position in the warp's sequence; stages waited for
    for (int ui = 0; ui < my_units; ++ui) {
        const int u = gw + ui * n_gw;
        float acc[2][T];
#pragma unroll
        for (int r = 0; r < 2; ++r)
#pragma unroll
            for (int t = 0; t < T; ++t) acc[r][t] = 0.f;
        for (int sg = 0; sg < n_seg; ++sg, ++f) {
            const int s = f % kGvStages;
            if (ok) {
                ok = __all_sync(0xffffffffu, mbar_wait_bounded(&full[s], (f / kGvStages) & 1));
                if (ok) consumed = f + 1;
            }
            if (ok) {
                const uint8_t* w0 = ring + s * stage_bytes + lane * 16;           // row j
                const uint8_t* w1 = w0 + seg_bytes;                              // row j + 64
                const uint8_t* xq = xs + sg * seg_bytes + lane * 16;
                // Two independent chains per row and token; the loads of a step are issued before its arithmetic.
#pragma unroll 2
                for (int c = 0; c < steps; ++c) {
                    const uint4 a = *reinterpret_cast<const uint4*>(w0 + c * 512);
                    const uint4 b = *reinterpret_cast<const uint4*>(w1 + c * 512);
                    const float a0 = bf16_lo(a.x), a1 = bf16_hi(a.x), a2 = bf16_lo(a.y), a3 = bf16_hi(a.y);
                    const float a4 = bf16_lo(a.z), a5 = bf16_hi(a.z), a6 = bf16_lo(a.w), a7 = bf16_hi(a.w);
                    const float b0 = bf16_lo(b.x), b1 = bf16_hi(b.x), b2 = bf16_lo(b.y), b3 = bf16_hi(b.y);
                    const float b4 = bf16_lo(b.z), b5 = bf16_hi(b.z), b6 = bf16_lo(b.w), b7 = bf16_hi(b.w);
#pragma unroll
                    for (int t = 0; t < T; ++t) {
                        const uint4 v = *reinterpret_cast<const uint4*>(xq + t * H * 2 + c * 512);
                        const float v0 = bf16_lo(v.x), v1 = bf16_hi(v.x), v2 = bf16_lo(v.y), v3 = bf16_hi(v.y);
                        const float v4 = bf16_lo(v.z), v5 = bf16_hi(v.z), v6 = bf16_lo(v.w), v7 = bf16_hi(v.w);
                        float e = a0 * v0, o = a1 * v1;
                        e = fmaf(a2, v2, e); o = fmaf(a3, v3, o);
                        e = fmaf(a4, v4, e); o = fmaf(a5, v5, o);
                        e = fmaf(a6, v6, e); o = fmaf(a7, v7, o);
                        acc[0][t] += e + o;
                        e = b0 * v0; o = b1 * v1;
                        e = fmaf(b2, v2, e); o = fmaf(b3, v3, o);
                        e = fmaf(b4, v4, e); o = fmaf(b5, v5, o);
                        e = fmaf(b6, v6, e); o = fmaf(b7, v7, o);
                        acc[1][t] += e + o;
                    }
                }
            }
            // Every lane has read the stage: it takes the segment that is two ahead in the warp's sequence.
            __syncwarp();
            if (lane == 0 && ok && issued < total) {
                issue(issued);
                ++issued;
            }
        }
        if (!ok) continue;
        // The pair's two dot products of every token: lane t finishes token t.
#pragma unroll
        for (int r = 0; r < 2; ++r)
#pragma unroll
            for (int t = 0; t < T; ++t) {
                float v = acc[r][t];
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
                acc[r][t] = v;
            }
        float lo = 0.f, hi = 0.f;
#pragma unroll
        for (int t = 0; t < T; ++t)
            if (lane == t) {
                lo = acc[0][t];
                hi = acc[1][t];
            }
        if (lane < T) {
            const int tok = lane;
            const int h = u >> 7, kv = (u >> 6) & 1, j = u & 63;
            lo = round_bf16(lo);
            hi = round_bf16(hi);
            if (kv == 0 && rotate) {
                const float cv = cs_s[tok * kProjHead + j], sv = cs_s[tok * kProjHead + 64 + j];
                const float a = lo, b = hi;
                lo = a * cv - b * sv;
                hi = b * cv + a * sv;
            }
            const __nv_bfloat16 blo = __float2bfloat16_rn(lo), bhi = __float2bfloat16_rn(hi);
            if (p.kv_new != nullptr) {
                __nv_bfloat16* d = p.kv_new + (static_cast<size_t>(tok) * p.nh_kv + h) * 256 + kv * 128 + j;
                d[0] = blo;
                d[64] = bhi;
            }
            const long long slot = my_slot;
            if (slot >= 0 && p.k_pool != nullptr) {
                if (slot < p.n_slots) {
                    __nv_bfloat16* d = (kv ? p.v_pool : p.k_pool) + (static_cast<size_t>(slot) * p.nh_kv + h) * 128 + j;
                    d[0] = blo;
                    d[64] = bhi;
                } else if (j == 0 && kv == 0) {
                    atomicOr(p.status, kStatusBadSlot);
                }
            }
        }
    }
    if (!ok && lane == 0) atomicOr(p.status, kStatusWaitTimeout | kStatusInProjLoad);
    // A copy that is still in flight when its CTA has gone would land in shared memory that another CTA may own by
    // then: wait (bounded) for every copy this warp issued and did not wait for.  Nothing to do on the normal path.
    if (lane == 0)
        for (int g = consumed; g < issued; ++g) mbar_wait_bounded(&full[g % kGvStages], (g / kGvStages) & 1);
}

}  // namespace dkv
