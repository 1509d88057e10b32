// K/V projection of a decode batch (at most 128 new tokens) on the 5th-generation tensor cores, sized to
// share an SM with the KV-streaming kernel.
//
// With only a handful of tokens the product is a stream over the weights, so the operands are swapped
// against dkv_proj.cuh: the 128 rows of Wk_h (then Wv_h) are the M side, the tokens the N side,
//
//   K_h^T[128 dims x N tokens] = Wk_h[128 x H] . X[N x H]^T        (bf16 x bf16 -> fp32 in TMEM)
//
// which shrinks the operands of one 64-column step to 32 KB of weights + N x 128 B of activations.  The ring is
// cut finer still: a stage holds ONE of the two weight chunks (Wk_h or Wv_h, 16 KB) with the X chunk it is
// multiplied by, so that within the same shared memory three to five stages are in flight while one is being
// multiplied (with two 34 KB stages only one was, and a short step ran at a third of the HBM rate).  128
// threads and under 96 registers per thread leave this CTA room beside a 16-warp streaming CTA (128 KB, 104
// registers), so the projection runs under the attention kernel instead of in front of it.
//
// Same contract as proj_rope_kernel (ProjParams): round to bf16, rotate K at the token's absolute
// position, round again, store to the pool and to kv_new (csrc/directKV_kernel.cuh:430-546 in the
// reference).  Split-K over gridDim.y; the CTA that arrives last adds the slices in a fixed order.
#pragma once

#include "dkv_proj.cuh"

namespace dkv {

constexpr int kPdMaxStages = 5;
constexpr int kPdWBytes    = kProjHead * kProjBK * 2;   // 16 KB: one 64-column chunk of Wk_h or Wv_h
constexpr int kPdRingBytes = 96 * 1024;                 // what the ring may take beside a streaming CTA
constexpr int kPdMaxTokens = 128;                       // tokens per CTA (N side of the product)
constexpr int kPdMaxBatch  = 512;                       // larger batches use the 128-token-tile kernel
constexpr int kPdChunkTok  = 32;                        // tokens per epilogue pass
constexpr int kPdAccStride = 132;                       // floats between token rows of the fp32 epilogue tile
constexpr int kPdCtrlBytes = 256;

__host__ __device__ constexpr int pd_padded_tokens(int T) { return (T + 15) / 16 * 16; }
__host__ __device__ constexpr int pd_stage_bytes(int n_pad) { return kPdWBytes + n_pad * 128; }   // one weight chunk + X chunk
__host__ __device__ constexpr int pd_stages(int n_pad) {
    return kPdRingBytes / pd_stage_bytes(n_pad) < kPdMaxStages ? kPdRingBytes / pd_stage_bytes(n_pad) : kPdMaxStages;
}
__host__ __device__ constexpr size_t pd_smem_bytes(int n_pad) {
    return static_cast<size_t>(pd_stages(n_pad)) * pd_stage_bytes(n_pad) + kPdCtrlBytes + 1024;
}
static_assert(pd_stages(kPdMaxTokens) >= 3 && pd_stages(16) == kPdMaxStages, "ring depth");
static_assert(2 * kPdChunkTok * kPdAccStride * 4 + kPdChunkTok * 512 <= pd_stages(16) * pd_stage_bytes(16) &&
              2 * kPdChunkTok * kPdAccStride * 4 + kPdChunkTok * 512 <= pd_stages(kPdMaxTokens) * pd_stage_bytes(kPdMaxTokens),
              "epilogue tiles must fit in the operand ring");
static_assert((2 * kPdMaxStages + 1) * 8 + 16 <= kPdCtrlBytes, "control block");

// grid (nh_kv, split_k, ceil(T / 128)), 128 threads: a CTA owns one KV head, one slice of the hidden dimension and
// up to 128 tokens.  tmX has box {64, min(128, T padded to 16)}; tmWk/tmWv box {64, 128}.
__global__ void __launch_bounds__(128, 5)   // at most 96 registers: the CTA must fit beside a streaming CTA
proj_rope_decode_kernel(const __grid_constant__ CUtensorMap tmX, const __grid_constant__ CUtensorMap tmWk,
                        const __grid_constant__ CUtensorMap tmWv, const ProjParams p) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const int tok_base = static_cast<int>(blockIdx.z) * kPdMaxTokens;
    const int T_cta = (p.T - tok_base) < kPdMaxTokens ? (p.T - tok_base) : kPdMaxTokens;   // tokens of this CTA
    const int n_pad = pd_padded_tokens(T_cta);                         // N of the product
    const int box_rows = p.T > kPdMaxTokens ? kPdMaxTokens : pd_padded_tokens(p.T);        // rows one TMA box of X brings
    const int stage_bytes = pd_stage_bytes(box_rows);
    const int n_stages = pd_stages(box_rows);
    const int vcol = n_pad <= 64 ? 64 : 128;             // TMEM column of the V accumulator
    const uint32_t tmem_cols = 2u * vcol;
    uint8_t* ctrl = smem + n_stages * stage_bytes;
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(ctrl);
    uint64_t* empty_bar = full_bar + kPdMaxStages;
    uint64_t* accum_bar = empty_bar + kPdMaxStages;
    uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(accum_bar + 1);
    volatile int* flags = reinterpret_cast<volatile int*>(tmem_holder + 1);  // [0] abort, [1] is_last

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int h = blockIdx.x, sp = blockIdx.y;
    const int nchunks = p.H / kProjBK;
    const int c0 = sp * p.chunks_per_split;
    const int c1 = (c0 + p.chunks_per_split < nchunks) ? c0 + p.chunks_per_split : nchunks;
    const int nloc = c1 - c0;

    if (tid == 0) {
        for (int s = 0; s < n_stages; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 1);
        }
        mbar_init(accum_bar, 1);
        flags[0] = 0;
        flags[1] = 0;
        fence_mbar_init();
        fence_proxy_async_smem();
        tma_prefetch_desc(&tmX);
        tma_prefetch_desc(&tmWk);
        tma_prefetch_desc(&tmWv);
    }
    if (warp == 1) {
        tmem_alloc(tmem_holder, tmem_cols);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_holder;

    if (warp == 0) {
        if (lane == 0) {
            // ---------------- TMA producer ----------------
            // Step j = 2 i + kv: chunk i of Wk_h (kv = 0) or Wv_h (kv = 1) and chunk i of X.
            for (int j = 0; j < 2 * nloc; ++j) {
                const int s = j % n_stages, round = j / n_stages;
                if (round > 0 && !mbar_wait_bounded(&empty_bar[s], (round - 1) & 1)) {
                    atomicOr(p.status, kStatusWaitTimeout | kStatusInProjLoad);
                    flags[0] = 1;
                    break;
                }
                uint8_t* st = smem + s * stage_bytes;
                mbar_arrive_expect_tx(&full_bar[s], static_cast<uint32_t>(stage_bytes));
                const int kc = (c0 + (j >> 1)) * kProjBK;
                tma_load_2d(st, (j & 1) ? &tmWv : &tmWk, &full_bar[s], kc, h * kProjHead);
                tma_load_2d(st + kPdWBytes, &tmX, &full_bar[s], kc, tok_base);   // rows past T read as zeros
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        if (lane == 0) {
            // ---------------- MMA issuer ----------------
            const uint32_t idesc = umma_idesc_bf16_f32(kProjHead, n_pad);
            bool ok = true;
            for (int j = 0; j < 2 * nloc; ++j) {
                const int s = j % n_stages, round = j / n_stages;
                if (!mbar_wait_bounded(&full_bar[s], round & 1)) {
                    atomicOr(p.status, kStatusWaitTimeout | kStatusInProjMma);
                    flags[0] = 1;
                    ok = false;
                    break;
                }
                tc_fence_after_sync();
                const uint32_t w_addr = smem_u32(smem + s * stage_bytes);
                const uint64_t w_desc = umma_desc_k_sw128(w_addr);
                const uint64_t x_desc = umma_desc_k_sw128(w_addr + kPdWBytes);
                const uint32_t d = tmem_base + ((j & 1) ? vcol : 0);
#pragma unroll
                for (int k4 = 0; k4 < kProjBK / 16; ++k4)
                    umma_bf16_ss(d, w_desc + 2 * k4, x_desc + 2 * k4, idesc, (j > 1 || k4 > 0) ? 1u : 0u);
                umma_commit(&empty_bar[s]);
            }
            if (ok) umma_commit(accum_bar);
            else mbar_arrive(accum_bar);
        }
        __syncwarp();
    }

    // ---------------- epilogue: all four warps; thread = output dimension ----------------
    bool ok = __all_sync(0xffffffffu, mbar_wait_bounded(accum_bar, 0));
    tc_fence_after_sync();
    if (!ok && lane == 0) {
        atomicOr(p.status, kStatusTmemTimeout | kStatusInProjMma);
        flags[0] = 1;
    }
    __syncthreads();
    const bool aborted = (flags[0] != 0);  // uniform across the CTA
    const uint32_t taddr = tmem_base + (static_cast<uint32_t>(warp * 32) << 16);
    const int npass = (T_cta + kPdChunkTok - 1) / kPdChunkTok;
    const int n_chunks = static_cast<int>(gridDim.z);
    const int unit = h * n_chunks + static_cast<int>(blockIdx.z);              // (head, token chunk) of this CTA
    const size_t slice_floats = static_cast<size_t>(2) * box_rows * kProjHead; // one (split, unit) slice: [2][box_rows][128]
    bool finalize = !aborted;

    if (!aborted && p.split_k > 1) {
        float* mine = p.splitk_scratch + (static_cast<size_t>(sp) * p.nh_kv * n_chunks + unit) * slice_floats + tid;
#pragma unroll 1
        for (int c = 0; c < npass; ++c) {
#pragma unroll 1
            for (int kv = 0; kv < 2; ++kv) {
                uint32_t r[32];
                tmem_ld_32x32(taddr + kv * vcol + c * kPdChunkTok, r);
                tmem_ld_wait();
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    const int tok = c * kPdChunkTok + i;
                    if (tok < T_cta) mine[(static_cast<size_t>(kv) * box_rows + tok) * kProjHead] = __uint_as_float(r[i]);
                }
            }
        }
        __threadfence();
        __syncthreads();
        if (tid == 0) {
            const unsigned int prev = atomicAdd(&p.tile_counters[unit], 1u);
            const int last = (prev == static_cast<unsigned int>(p.split_k - 1));
            if (last) p.tile_counters[unit] = 0u;  // ready for the next launch
            flags[1] = last;
        }
        __syncthreads();
        finalize = (flags[1] != 0);
        if (finalize) __threadfence();
    }

    float* sacc = reinterpret_cast<float*>(smem);                                  // [2][32][132] fp32
    uint8_t* stage_out = smem + 2 * kPdChunkTok * kPdAccStride * 4;                // [32][512 B]: K row | V row
    if (finalize) {
#pragma unroll 1
        for (int c = 0; c < npass; ++c) {
            const int tok0 = c * kPdChunkTok;
            const int rows = (T_cta - tok0) < kPdChunkTok ? (T_cta - tok0) : kPdChunkTok;
            if (p.split_k == 1) {
#pragma unroll 1
                for (int kv = 0; kv < 2; ++kv) {
                    uint32_t r[32];
                    tmem_ld_32x32(taddr + kv * vcol + tok0, r);
                    tmem_ld_wait();
#pragma unroll
                    for (int i = 0; i < 32; ++i) sacc[(kv * kPdChunkTok + i) * kPdAccStride + tid] = __uint_as_float(r[i]);
                }
            } else {
                const float* slice0 = p.splitk_scratch + static_cast<size_t>(unit) * slice_floats;
                const size_t split_stride = static_cast<size_t>(p.nh_kv) * n_chunks * slice_floats;
                for (int idx = tid; idx < 2 * rows * 32; idx += 128) {
                    const int c4 = idx & 31, r = (idx >> 5) % rows, kv = (idx >> 5) / rows;
                    const float* src = slice0 + (static_cast<size_t>(kv) * box_rows + tok0 + r) * kProjHead + c4 * 4;
                    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
                    for (int s2 = 0; s2 < p.split_k; ++s2) {
                        const float4 f = __ldcg(reinterpret_cast<const float4*>(src + s2 * split_stride));
                        acc.x += f.x;
                        acc.y += f.y;
                        acc.z += f.z;
                        acc.w += f.w;
                    }
                    *reinterpret_cast<float4*>(sacc + (kv * kPdChunkTok + r) * kPdAccStride + c4 * 4) = acc;
                }
            }
            __syncthreads();
            // Round, rotate K (dims d and d + 64 together), round again; V is rounded once.
            for (int r = 0; r < rows; ++r) {
                const int tok = tok_base + tok0 + r;       // row of X / position in the batch
                if (tid < 64) {
                    float lo = round_bf16(sacc[r * kPdAccStride + tid]);
                    float hi = round_bf16(sacc[r * kPdAccStride + tid + 64]);
                    if (p.cos_sin != nullptr && proj_has_pos(p)) {
                        const int pos = proj_tok_pos(p, tok);
                        if (pos >= 0 && pos < p.max_pos) {
                            const float* cs = p.cos_sin + static_cast<size_t>(pos) * kProjHead;
                            const float cv = __ldg(cs + tid), sv = __ldg(cs + 64 + tid);
                            const float a = lo, b = hi;
                            lo = a * cv - b * sv;
                            hi = b * cv + a * sv;
                        } else if (tid == 0) {
                            atomicOr(p.status, kStatusBadPosition);
                        }
                    }
                    *reinterpret_cast<__nv_bfloat16*>(stage_out + r * 512 + tid * 2) = __float2bfloat16_rn(lo);
                    *reinterpret_cast<__nv_bfloat16*>(stage_out + r * 512 + 128 + tid * 2) = __float2bfloat16_rn(hi);
                } else {
                    const int d = (tid - 64) * 2;
                    const float* src = sacc + (kPdChunkTok + r) * kPdAccStride + d;
                    *reinterpret_cast<uint32_t*>(stage_out + r * 512 + 256 + d * 2) = pack_bf16x2(src[0], src[1]);
                }
            }
            __syncthreads();
            // Coalesced copy-out: one warp writes one token's 256-byte K row and 256-byte V row.
            for (int r = warp; r < rows; r += 4) {
                const int tok = tok_base + tok0 + r;       // row of X / position in the batch
                const uint4 w = *reinterpret_cast<const uint4*>(stage_out + r * 512 + lane * 16);
                if (p.kv_new != nullptr)
                    *reinterpret_cast<uint4*>(p.kv_new + (static_cast<size_t>(tok) * p.nh_kv + h) * 256 + lane * 8) = w;
                const long long slot = proj_tok_slot(p, tok);
                if (slot >= 0 && p.k_pool != nullptr) {
                    if (slot < p.n_slots) {
                        __nv_bfloat16* dst = (lane < 16 ? p.k_pool : p.v_pool) +
                                             (static_cast<size_t>(slot) * p.nh_kv + h) * 128 + (lane & 15) * 8;
                        *reinterpret_cast<uint4*>(dst) = w;
                    } else if (lane == 0) {
                        atomicOr(p.status, kStatusBadSlot);
                    }
                }
            }
            __syncthreads();
        }
    }
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem_base, tmem_cols);
}

}  // namespace dkv
