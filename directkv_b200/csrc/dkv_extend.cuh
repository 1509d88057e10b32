// Extend / chunked-prefill attention on the 5th-generation tensor cores.
//
// The new rows of a request attend its past rows plus their own causal prefix
// (mask: key j visible to new row i iff j <= seqlen_past + i; reference
// directkv/directkv_backend.py:887, csrc/directKV_kernel.cuh:654-678).  One CTA owns 128 query rows -
// G query heads of one KV head times 128/G consecutive new tokens, so a K/V tile is read once per
// group - and walks the keys in tiles of 128:
//
//   S = Q K^T          tcgen05.mma  M=128 N=128 K=128  (bf16, fp32 in TMEM columns [0,128))
//   P = exp2(S*c - m)  row-per-thread softmax from TMEM, P stored bf16 into swizzled smem
//   T = P V            tcgen05.mma  M=128 N=128 K=128  (V consumed MN-major straight from the
//                      [token][d] tile TMA loaded; TMEM columns [128,256))
//   O = O*alpha + T    fp32 in registers (128 per thread)
//
// K/V tiles arrive by TMA (128-byte swizzle) into a two-stage ring, the next tile is in flight
// while the current one is processed.  All waits are bounded.
#pragma once

#include "dkv_common.cuh"

namespace dkv {

constexpr int kExtTile = 128;                        // query rows per CTA and keys per tile
constexpr int kExtHalfBytes = kExtTile * 128;        // one [128 rows x 64 bf16] swizzled block: 16 KB
constexpr int kExtTileBytes = 2 * kExtHalfBytes;     // [128 x 128] bf16: 32 KB
constexpr int kExtStages = 2;
constexpr int kExtSmem = kExtTileBytes /*Q*/ + kExtTileBytes /*P*/ + kExtStages * 2 * kExtTileBytes /*K,V*/ + 1024;

struct ExtendParams {
    const int* vrow;            // [B] pool / staging row of request b (nullptr: b)
    const int* n_past_blocks;   // device scalar: seqlen_past = n_past_blocks[0] * 64, or nullptr
    int seqlen_past;            // used when n_past_blocks == nullptr
    int S_new;
    int nh_q, nh_kv;
    int G;                      // query heads per CTA (power of two dividing g_total)
    int g_total, nsub;          // nh_q / nh_kv, g_total / G
    long long row_stride;       // slots per row of the K/V tensor the maps describe
    int is_causal;
    float scale_log2;
    __nv_bfloat16* out;         // [B, S_new, nh_q, 128]
    unsigned int* status;
    // Ragged batch (extend_attn_pp_kernel only): blockIdx.y indexes a work list of (request, query-tile pair)
    // sorted longest first; every request has its own number of new rows, past length, first row in the packed
    // Q / O tensors and first slot of its K/V rows.  nullptr: uniform batch described by the fields above.
    const int2* items;
    const int* r_s_new;
    const int* r_past;
    const int* r_q_row0;
    const int* r_slot0;
};

// Descriptor of a [64 x 8]-element MN-major, 128-byte-swizzled atom grid: rows (K index) are 128 bytes apart,
// groups of 8 rows are 1024 bytes apart (stride byte offset), the next 64 elements along MN start
// `mn_stride` bytes further (leading byte offset).
__device__ __forceinline__ uint64_t umma_desc_mn_sw128(uint32_t smem_addr, uint32_t mn_stride) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((smem_addr & 0x3ffffu) >> 4);
    d |= static_cast<uint64_t>((mn_stride >> 4) & 0x3fffu) << 16;
    d |= static_cast<uint64_t>(1024 >> 4) << 32;
    d |= static_cast<uint64_t>(1) << 46;
    d |= static_cast<uint64_t>(2) << 61;
    return d;
}

__global__ void __launch_bounds__(128, 1)
extend_attn_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                   const __grid_constant__ CUtensorMap tmV, const ExtendParams p) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* sQ = smem;
    uint8_t* sP = sQ + kExtTileBytes;
    uint8_t* sKV = sP + kExtTileBytes;                       // stage s: K at +s*64K, V at +s*64K + 32K
    uint8_t* ctrl = sKV + kExtStages * 2 * kExtTileBytes;
    uint64_t* bar_q = reinterpret_cast<uint64_t*>(ctrl);
    uint64_t* bar_kv = bar_q + 1;                            // [kExtStages]
    uint64_t* bar_s = bar_kv + kExtStages;
    uint64_t* bar_o = bar_s + 1;
    uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(bar_o + 1);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int G = p.G, TQ = kExtTile / G;
    const int qt = blockIdx.x, b = blockIdx.z;
    const int h = blockIdx.y / p.nsub, sub = blockIdx.y % p.nsub;   // KV head, group of G query heads
    const int qhead0 = h * p.g_total + sub * G;
    const int past = p.n_past_blocks ? p.n_past_blocks[0] * 64 : p.seqlen_past;
    const int q0 = qt * TQ;                                   // first new-token index of this CTA
    const int row_slot0 = static_cast<int>(static_cast<long long>(p.vrow ? p.vrow[b] : b) * p.row_stride);
    const int s_total = past + p.S_new;
    int kv_end = p.is_causal ? past + q0 + TQ : s_total;      // keys this CTA can see: [0, kv_end)
    if (kv_end > s_total) kv_end = s_total;
    const int n_tiles = (kv_end + kExtTile - 1) / kExtTile;

    if (tid == 0) {
        mbar_init(bar_q, 1);
        for (int s = 0; s < kExtStages; ++s) mbar_init(&bar_kv[s], 1);
        mbar_init(bar_s, 1);
        mbar_init(bar_o, 1);
        fence_mbar_init();
        fence_proxy_async_smem();
        tma_prefetch_desc(&tmQ);
        tma_prefetch_desc(&tmK);
        tma_prefetch_desc(&tmV);
    }
    if (warp == 1) {
        tmem_alloc(tmem_holder, 256);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_holder;

    auto issue_kv = [&](int tile, int stage) {
        uint8_t* k_dst = sKV + stage * 2 * kExtTileBytes;
        uint8_t* v_dst = k_dst + kExtTileBytes;
        mbar_arrive_expect_tx(&bar_kv[stage], 2 * kExtTileBytes);
        const int slot = row_slot0 + tile * kExtTile;
        tma_load_3d(k_dst, &tmK, &bar_kv[stage], 0, h, slot);
        tma_load_3d(k_dst + kExtHalfBytes, &tmK, &bar_kv[stage], 64, h, slot);
        tma_load_3d(v_dst, &tmV, &bar_kv[stage], 0, h, slot);
        tma_load_3d(v_dst + kExtHalfBytes, &tmV, &bar_kv[stage], 64, h, slot);
    };

    if (tid == 0) {
        // Q rows r = t * G + g come as a (d, head, token) box: G heads of TQ tokens.
        mbar_arrive_expect_tx(bar_q, kExtTileBytes);
        tma_load_3d(sQ, &tmQ, bar_q, 0, qhead0, b * p.S_new + q0);
        tma_load_3d(sQ + kExtHalfBytes, &tmQ, bar_q, 64, qhead0, b * p.S_new + q0);
        if (n_tiles > 0) issue_kv(0, 0);
    }

    const int row = warp * 32 + lane;                 // TMEM lane == query row of this thread
    const int my_tok = q0 + row / G;                  // new-token index of the row
    const int my_limit = p.is_causal ? past + my_tok : s_total - 1;   // last visible key
    const uint32_t taddr = tmem_base + (static_cast<uint32_t>(warp * 32) << 16);
    constexpr uint32_t idesc_qk = umma_idesc_bf16_f32(kExtTile, kExtTile);
    constexpr uint32_t idesc_pv = umma_idesc_bf16_f32(kExtTile, kExtTile) | (1u << 16);   // B is MN-major

    float O[128];
#pragma unroll
    for (int i = 0; i < 128; ++i) O[i] = 0.f;
    float m = -INFINITY, l = 0.f;
    bool ok = true;

    if (!mbar_wait_bounded(bar_q, 0)) ok = false;

    for (int it = 0; it < n_tiles; ++it) {
        const int stage = it & 1;
        const uint8_t* sK = sKV + stage * 2 * kExtTileBytes;
        uint8_t* sV = const_cast<uint8_t*>(sK) + kExtTileBytes;
        if (tid == 0 && it + 1 < n_tiles) issue_kv(it + 1, stage ^ 1);
        if (!mbar_wait_bounded(&bar_kv[stage], (it >> 1) & 1)) ok = false;

        // Rows of the tile past the request's last token may hold anything (another request's data, or
        // never-written memory): V must be finite there because P (zero) still multiplies it.
        const int tile_valid = s_total - it * kExtTile;
        if (tile_valid < kExtTile) {
            for (int idx = tid; idx < (kExtTile - tile_valid) * 16; idx += 128) {
                const int r = tile_valid + idx / 16, c = idx % 16;     // 16-byte chunk c of row r (both halves)
                *reinterpret_cast<uint4*>(sV + (c >> 3) * kExtHalfBytes + r * 128 + ((c & 7) << 4)) = make_uint4(0, 0, 0, 0);
            }
            fence_proxy_async_smem();
        }
        tc_fence_before_sync();
        ok = __syncthreads_and(ok);
        if (!ok) break;
        tc_fence_after_sync();

        // ---- S = Q K^T ----
        if (tid == 0) {
            const uint32_t qa = smem_u32(sQ), ka = smem_u32(sK);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const uint32_t off = (j >> 2) * kExtHalfBytes + (j & 3) * 32;
                umma_bf16_ss(tmem_base, umma_desc_k_sw128(qa + off), umma_desc_k_sw128(ka + off), idesc_qk, j > 0 ? 1u : 0u);
            }
            umma_commit(bar_s);
        }
        if (!mbar_wait_bounded(bar_s, it & 1)) ok = false;
        tc_fence_after_sync();

        // ---- softmax of this thread's row; P -> smem (K-major, swizzled like a TMA tile) ----
        // Two passes over the 128 scores in TMEM (row maximum, then probabilities) keep only 32 of them
        // in registers at a time next to the 128 output accumulators.
        const int col0 = it * kExtTile;
        float m_new = m;
#pragma unroll 1
        for (int c = 0; c < 4; ++c) {
            uint32_t r[32];
            tmem_ld_32x32(taddr + c * 32, r);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) {
                const int col = col0 + c * 32 + i;
                if (col <= my_limit) m_new = fmaxf(m_new, __uint_as_float(r[i]) * p.scale_log2);
            }
        }
        const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
        const float alpha = exp2f(m - m_use);
        float psum = 0.f;
#pragma unroll 1
        for (int c = 0; c < 4; ++c) {
            uint32_t r[32];
            tmem_ld_32x32(taddr + c * 32, r);
            tmem_ld_wait();
#pragma unroll
            for (int q8 = 0; q8 < 4; ++q8) {              // 16-byte chunk = 8 probabilities
                float pv[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const int col = col0 + c * 32 + q8 * 8 + i;
                    pv[i] = (col <= my_limit) ? exp2f(__uint_as_float(r[q8 * 8 + i]) * p.scale_log2 - m_use) : 0.f;
                    psum += pv[i];
                }
                uint4 w;
                w.x = pack_bf16x2(pv[0], pv[1]);
                w.y = pack_bf16x2(pv[2], pv[3]);
                w.z = pack_bf16x2(pv[4], pv[5]);
                w.w = pack_bf16x2(pv[6], pv[7]);
                const int c8 = c * 4 + q8;                 // chunk index within the 128-key row
                const int half = c8 >> 3, ch = c8 & 7;
                *reinterpret_cast<uint4*>(sP + half * kExtHalfBytes + row * 128 + ((ch ^ (row & 7)) << 4)) = w;
            }
        }
        l = l * alpha + psum;
        m = m_new;
#pragma unroll
        for (int i = 0; i < 128; ++i) O[i] *= alpha;
        fence_proxy_async_smem();
        tc_fence_before_sync();
        ok = __syncthreads_and(ok);
        if (!ok) break;
        tc_fence_after_sync();

        // ---- T = P V ----
        if (tid == 0) {
            const uint32_t pa = smem_u32(sP), va = smem_u32(sV);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const uint32_t aoff = (j >> 2) * kExtHalfBytes + (j & 3) * 32;   // 16 keys along K of P
                const uint32_t boff = j * 16 * 128;                               // 16 key rows of V
                umma_bf16_ss(tmem_base + 128, umma_desc_k_sw128(pa + aoff), umma_desc_mn_sw128(va + boff, kExtHalfBytes),
                             idesc_pv, j > 0 ? 1u : 0u);
            }
            umma_commit(bar_o);
        }
        if (!mbar_wait_bounded(bar_o, it & 1)) ok = false;
        tc_fence_after_sync();
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            uint32_t r[32];
            tmem_ld_32x32(taddr + 128 + c * 32, r);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) O[c * 32 + i] += __uint_as_float(r[i]);
        }
    }

    ok = __syncthreads_and(ok);
    if (!ok) {
        if (tid == 0) atomicOr(p.status, kStatusWaitTimeout | kStatusInExtend);
    } else if (my_tok < p.S_new) {
        const float inv = l > 0.f ? 1.f / l : 0.f;
        const int g = row % G;
        __nv_bfloat16* dst = p.out + ((static_cast<long long>(b) * p.S_new + my_tok) * p.nh_q + qhead0 + g) * 128;
#pragma unroll
        for (int c = 0; c < 16; ++c) {
            uint4 w;
            w.x = pack_bf16x2(O[c * 8 + 0] * inv, O[c * 8 + 1] * inv);
            w.y = pack_bf16x2(O[c * 8 + 2] * inv, O[c * 8 + 3] * inv);
            w.z = pack_bf16x2(O[c * 8 + 4] * inv, O[c * 8 + 5] * inv);
            w.w = pack_bf16x2(O[c * 8 + 6] * inv, O[c * 8 + 7] * inv);
            *reinterpret_cast<uint4*>(dst + c * 8) = w;
        }
    }
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem_base, 256);
}

}  // namespace dkv
