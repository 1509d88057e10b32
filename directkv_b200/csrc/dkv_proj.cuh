// K/V projection of new tokens on the 5th-generation tensor cores, with the Neox rotation of K
// and the write-back to the KV pool fused into the epilogue.
//
//   [K_h | V_h](t, :) = X(t, :) . [Wk_h ; Wv_h]^T      (bf16 x bf16 -> fp32 in TMEM)
//
// restates what the reference computes in csrc/directKV_kernel.cuh:430-546 (project, round to
// bf16, rotate K at the token's absolute position, round again, store to the pool), but over the
// FULL hidden size (the reference contracts only its first 128 columns).
//
// One CTA owns a 128-token x 256-column tile (one KV head: 128 K columns then 128 V columns)
// and a slice of the hidden dimension.  TMA brings 64-column chunks of X, Wk_h and Wv_h into a
// 128-byte-swizzled ring; one thread issues tcgen05.mma (M=128, N=256, K=16) into a 256-column
// TMEM accumulator.  With split-K every CTA stores its fp32 tile to scratch and the CTA that
// arrives last adds the slices in a fixed order, so results do not depend on scheduling.
#pragma once

#include "dkv_common.cuh"

namespace dkv {

constexpr int kProjBM        = 128;                   // tokens per tile (TMEM lanes)
constexpr int kProjBN        = 256;                   // K_h (128) | V_h (128)
constexpr int kProjBK        = 64;                    // hidden columns per stage (128 bytes of bf16)
constexpr int kProjABytes    = kProjBM * kProjBK * 2; // 16 KB
constexpr int kProjBBytes    = kProjBN * kProjBK * 2; // 32 KB
constexpr int kProjStage     = kProjABytes + kProjBBytes;
constexpr int kProjTmemCols  = 256;
constexpr int kProjAccStride = kProjBN + 4;           // floats between rows of the split-K sum tile
constexpr int kProjHead      = 128;                   // head dimension (rows of Wk_h / Wv_h)

// Where the one new token of each request of a DECODE step goes, worked out by the projection itself from the
// call's own arguments (tok_pos / tok_slot are nullptr then): the kernel reads nothing that the prep kernel
// writes, so the two start together instead of one after the other.  Same arithmetic as attn_prep_kernel.
struct DecodePlace {
    const int* seq_lens;           // [T] tokens of request t including the new one; nullptr: not a decode step
    const int* page_table;         // [rows, pt_stride] or nullptr (contiguous rows)
    const int* row_map;            // [T] or nullptr
    const int* pos_offset;         // [T] added to the RoPE position, or nullptr
    int pt_stride, pt_rows, page_size, page_shift;
    long long row_stride;
    int save;                      // store the token to the pool
};

struct ProjParams {
    int T;                         // tokens (rows of X)
    int H;                         // hidden size, multiple of 64
    int nh_kv;
    int split_k;                   // gridDim.z
    int chunks_per_split;          // 64-column chunks each split handles
    const int* tok_pos;            // [T] absolute position for RoPE, or nullptr
    const int* tok_slot;           // [T] pool slot to store to (< 0: none), or nullptr
    const float* cos_sin;          // [max_pos, 128] fp32 (cos | sin), or nullptr = no rotation
    int max_pos;
    __nv_bfloat16* k_pool;         // [n_slots, nh_kv, 128] (host-mapped or HBM), may be nullptr
    __nv_bfloat16* v_pool;
    long long n_slots;
    __nv_bfloat16* kv_new;         // [T, nh_kv, 2, 128] bf16 in HBM, or nullptr
    float* splitk_scratch;         // [split_k, tilesM, nh_kv, 128, 256] fp32
    unsigned int* tile_counters;   // [tilesM * nh_kv], zero between launches
    unsigned int* status;
    DecodePlace place;
};

__device__ __forceinline__ bool proj_has_pos(const ProjParams& p) {
    return p.tok_pos != nullptr || p.place.seq_lens != nullptr;
}

// Absolute (RoPE) position of token `tok`.
__device__ __forceinline__ int proj_tok_pos(const ProjParams& p, int tok) {
    if (p.tok_pos != nullptr) return p.tok_pos[tok];
    return p.place.seq_lens[tok] - 1 + (p.place.pos_offset ? p.place.pos_offset[tok] : 0);
}

// Pool slot token `tok` is stored to, or -1.
__device__ __forceinline__ long long proj_tok_slot(const ProjParams& p, int tok) {
    if (p.tok_slot != nullptr) return p.tok_slot[tok];
    const DecodePlace& d = p.place;
    if (d.seq_lens == nullptr || !d.save) return -1;
    const int pos = d.seq_lens[tok] - 1;
    if (pos < 0) return -1;
    const int row = d.row_map ? d.row_map[tok] : tok;
    if (d.page_table == nullptr) return static_cast<long long>(row) * d.row_stride + pos;
    const int pg = pos >> d.page_shift;
    if (pg >= d.pt_stride || row < 0 || (d.pt_rows > 0 && row >= d.pt_rows)) {
        atomicOr(p.status, kStatusBadPage);           // the token is not stored
        return -1;
    }
    return (static_cast<long long>(d.page_table[static_cast<long long>(row) * d.pt_stride + pg]) << d.page_shift) +
           (pos & (d.page_size - 1));
}

// MT = 128-token sub-tiles per CTA (1 or 2).  With two, a stage holds 32 KB of X next to the same 32 KB of
// weights and both halves of the 512 TMEM columns are used, so the weights cross L2 -> SM once per 256 tokens:
// at prefill sizes the kernel is bound by that traffic, not by the tensor pipe.
template <int NST, int MT>
__global__ void __launch_bounds__(128, 1)
proj_rope_kernel(const __grid_constant__ CUtensorMap tmX, const __grid_constant__ CUtensorMap tmWk,
                 const __grid_constant__ CUtensorMap tmWv, const ProjParams p) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    // The swizzled operand tiles need 1024-byte alignment.
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    // Control words sit behind the area the epilogue re-uses (sum tile + output staging = 198,656 B).
    constexpr int kStage = MT * kProjABytes + kProjBBytes;
    uint8_t* ctrl = smem + NST * kStage + 4096;
    static_assert(NST * kStage + 4096 >= kProjBM * kProjAccStride * 4 + kProjBM * 512, "epilogue tiles overlap the control words");
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(ctrl);
    uint64_t* empty_bar = full_bar + NST;
    uint64_t* accum_bar = empty_bar + NST;
    uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(accum_bar + 1);
    volatile int* flags = reinterpret_cast<volatile int*>(tmem_holder + 1);  // [0] abort, [1] is_last

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int h = blockIdx.x, sp = blockIdx.z;
    const int n_mtiles = static_cast<int>(gridDim.y) * MT;            // 128-token tiles over all CTAs
    const int nchunks = p.H / kProjBK;
    const int c0 = sp * p.chunks_per_split;
    const int c1 = (c0 + p.chunks_per_split < nchunks) ? c0 + p.chunks_per_split : nchunks;
    const int nloc = c1 - c0;

    if (tid == 0) {
#pragma unroll
        for (int s = 0; s < NST; ++s) {
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
        tmem_alloc(tmem_holder, MT * kProjTmemCols);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_holder;

    if (warp == 0) {
        if (lane == 0) {
            // ---------------- TMA producer ----------------
            for (int i = 0; i < nloc; ++i) {
                const int s = i % NST;
                if (i >= NST && !mbar_wait_bounded(&empty_bar[s], ((i / NST) - 1) & 1)) {
                    atomicOr(p.status, kStatusWaitTimeout | kStatusInProjLoad);
                    flags[0] = 1;
                    break;
                }
                uint8_t* st = smem + s * kStage;
                mbar_arrive_expect_tx(&full_bar[s], kStage);
                const int kc = (c0 + i) * kProjBK;
                tma_load_2d(st, &tmX, &full_bar[s], kc, static_cast<int>(blockIdx.y) * MT * kProjBM);   // box of MT * 128 rows
                tma_load_2d(st + MT * kProjABytes, &tmWk, &full_bar[s], kc, h * kProjHead);
                tma_load_2d(st + MT * kProjABytes + kProjBBytes / 2, &tmWv, &full_bar[s], kc, h * kProjHead);
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        if (lane == 0) {
            // ---------------- MMA issuer ----------------
            constexpr uint32_t idesc = umma_idesc_bf16_f32(kProjBM, kProjBN);
            bool ok = true;
            for (int i = 0; i < nloc; ++i) {
                const int s = i % NST;
                if (!mbar_wait_bounded(&full_bar[s], (i / NST) & 1)) {
                    atomicOr(p.status, kStatusWaitTimeout | kStatusInProjMma);
                    flags[0] = 1;
                    ok = false;
                    break;
                }
                tc_fence_after_sync();
                const uint32_t a_addr = smem_u32(smem + s * kStage);
                const uint64_t a_desc = umma_desc_k_sw128(a_addr);
                const uint64_t b_desc = umma_desc_k_sw128(a_addr + MT * kProjABytes);
#pragma unroll
                for (int k4 = 0; k4 < kProjBK / 16; ++k4)
#pragma unroll
                    for (int m = 0; m < MT; ++m)
                        umma_bf16_ss(tmem_base + m * kProjTmemCols, a_desc + (m * kProjABytes) / 16 + 2 * k4, b_desc + 2 * k4, idesc,
                                     (i > 0 || k4 > 0) ? 1u : 0u);
                umma_commit(&empty_bar[s]);  // the stage is free once these MMAs have read it
            }
            if (ok) umma_commit(accum_bar);
            else mbar_arrive(accum_bar);
        }
        __syncwarp();
    }

    // ---------------- epilogue: all four warps ----------------
    bool ok = __all_sync(0xffffffffu, mbar_wait_bounded(accum_bar, 0));
    tc_fence_after_sync();
    if (!ok && lane == 0) {
        atomicOr(p.status, kStatusTmemTimeout | kStatusInProjMma);
        flags[0] = 1;
    }
    __syncthreads();
    const bool aborted = (flags[0] != 0);  // uniform across the CTA

    const int row = warp * 32 + lane;
#pragma unroll 1
    for (int msub = 0; msub < MT; ++msub) {
    const int mt = static_cast<int>(blockIdx.y) * MT + msub;          // 128-token tile of this pass
    if (mt * kProjBM >= p.T) break;                                   // CTA-uniform
    const int token = mt * kProjBM + row;
    const uint32_t taddr = tmem_base + (static_cast<uint32_t>(warp * 32) << 16) + msub * kProjTmemCols;
    uint8_t* stage_out = smem;  // [128 rows][512 B], 16-byte chunks XOR-swizzled by row (after the sum tile with split-K)
    bool finalize = !aborted;

    if (!aborted && p.split_k > 1) {
        // Dump this CTA's fp32 tile, then let the CTA that arrives last combine all slices.
        float* mine = p.splitk_scratch +
                      ((static_cast<size_t>(sp) * n_mtiles + mt) * p.nh_kv + h) * (kProjBM * kProjBN) +
                      static_cast<size_t>(row) * kProjBN;
#pragma unroll 1
        for (int c = 0; c < kProjBN / 32; ++c) {
            uint32_t r[32];
            tmem_ld_32x32(taddr + c * 32, r);
            tmem_ld_wait();
            if (token < p.T) {
#pragma unroll
                for (int i = 0; i < 32; i += 4)
                    *reinterpret_cast<uint4*>(mine + c * 32 + i) = make_uint4(r[i], r[i + 1], r[i + 2], r[i + 3]);
            }
        }
        __threadfence();
        __syncthreads();
        if (tid == 0) {
            const unsigned int prev = atomicAdd(&p.tile_counters[mt * p.nh_kv + h], 1u);
            const int last = (prev == static_cast<unsigned int>(p.split_k - 1));
            if (last) p.tile_counters[mt * p.nh_kv + h] = 0u;  // ready for the next launch
            flags[1] = last;
        }
        __syncthreads();
        finalize = (flags[1] != 0);
        if (finalize) __threadfence();
    }

    // Split-K: all threads of the last CTA add the slices (fixed order s = 0, 1, ...) into an fp32
    // tile in shared memory; rows are 260 floats apart so that the row-per-thread reads below do not
    // collide on banks.
    float* sacc = reinterpret_cast<float*>(smem);
    if (finalize && p.split_k > 1) {
        const int rows_valid = (p.T - mt * kProjBM) < kProjBM ? (p.T - mt * kProjBM) : kProjBM;
        const float* tile0 = p.splitk_scratch + ((static_cast<size_t>(mt)) * p.nh_kv + h) * (kProjBM * kProjBN);
        const size_t slice_stride = static_cast<size_t>(n_mtiles) * p.nh_kv * (kProjBM * kProjBN);
        for (int idx = tid; idx < rows_valid * (kProjBN / 4); idx += 128) {
            const int r = idx / (kProjBN / 4), c4 = idx % (kProjBN / 4);
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
            for (int s2 = 0; s2 < p.split_k; ++s2) {
                const float4 f = __ldcg(reinterpret_cast<const float4*>(tile0 + s2 * slice_stride + r * kProjBN + c4 * 4));
                acc.x += f.x;
                acc.y += f.y;
                acc.z += f.z;
                acc.w += f.w;
            }
            *reinterpret_cast<float4*>(sacc + r * kProjAccStride + c4 * 4) = acc;
        }
        stage_out = smem + kProjBM * kProjAccStride * 4;
        __syncthreads();
    }

    // tcgen05.ld is warp-collective: a warp takes this branch as a whole (the condition is
    // warp-uniform) and lanes past the last token only skip the global-memory accesses.
    const bool warp_has_tokens = (mt * kProjBM + warp * 32) < p.T;
    const bool lane_valid = token < p.T;
    if (finalize && warp_has_tokens) {
        auto load32 = [&](int col, float (&v)[32]) {
            if (p.split_k == 1) {
                uint32_t r[32];
                tmem_ld_32x32(taddr + col, r);
                tmem_ld_wait();
#pragma unroll
                for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
            } else {
                const float* src = sacc + row * kProjAccStride + col;
#pragma unroll
                for (int i = 0; i < 32; i += 4) {
                    const float4 f = *reinterpret_cast<const float4*>(src + i);
                    v[i] = f.x;
                    v[i + 1] = f.y;
                    v[i + 2] = f.z;
                    v[i + 3] = f.w;
                }
            }
        };
        auto store32 = [&](int col, const float (&v)[32]) {
            // 32 bf16 = 64 bytes = chunks col/8 .. col/8 + 3 of this row
#pragma unroll
            for (int q4 = 0; q4 < 4; ++q4) {
                uint4 w;
                w.x = pack_bf16x2(v[8 * q4 + 0], v[8 * q4 + 1]);
                w.y = pack_bf16x2(v[8 * q4 + 2], v[8 * q4 + 3]);
                w.z = pack_bf16x2(v[8 * q4 + 4], v[8 * q4 + 5]);
                w.w = pack_bf16x2(v[8 * q4 + 6], v[8 * q4 + 7]);
                const int chunk = (col >> 3) + q4;
                *reinterpret_cast<uint4*>(stage_out + row * 512 + ((chunk ^ (row & 31)) << 4)) = w;
            }
        };

        int pos = -1;
        if (lane_valid && p.cos_sin != nullptr && proj_has_pos(p)) {
            pos = proj_tok_pos(p, token);
            if (pos < 0 || pos >= p.max_pos) {
                atomicOr(p.status, kStatusBadPosition);
                pos = -1;
            }
        }
        // K: columns d and d + 64 rotate together.
#pragma unroll 1
        for (int c = 0; c < 2; ++c) {
            float lo[32], hi[32];
            load32(32 * c, lo);
            load32(64 + 32 * c, hi);
#pragma unroll
            for (int i = 0; i < 32; ++i) {
                lo[i] = round_bf16(lo[i]);
                hi[i] = round_bf16(hi[i]);
            }
            if (pos >= 0) {
                const float* cs = p.cos_sin + static_cast<size_t>(pos) * kProjHead;
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    const float cv = __ldg(cs + 32 * c + i), sv = __ldg(cs + 64 + 32 * c + i);
                    const float a = lo[i], b = hi[i];
                    lo[i] = a * cv - b * sv;
                    hi[i] = b * cv + a * sv;
                }
            }
            store32(32 * c, lo);
            store32(64 + 32 * c, hi);
        }
        // V
#pragma unroll 1
        for (int c = 0; c < 4; ++c) {
            float v[32];
            load32(128 + 32 * c, v);
            store32(128 + 32 * c, v);
        }
    }
    tc_fence_before_sync();
    __syncthreads();

    if (finalize) {
        // Coalesced copy-out: one warp writes one token's 256-byte K row and 256-byte V row.
        for (int r = warp; r < kProjBM; r += 4) {
            const int tok = mt * kProjBM + r;
            if (tok >= p.T) break;
            const uint4 w = *reinterpret_cast<const uint4*>(stage_out + r * 512 + ((lane ^ (r & 31)) << 4));
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
    }
    __syncthreads();     // the next pass re-uses the shared-memory tiles and the flags
    if (tid == 0) flags[1] = 0;
    }
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem_base, MT * kProjTmemCols);
}

}  // namespace dkv
