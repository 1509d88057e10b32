// Extend / chunked-prefill attention, two query tiles per CTA in ping-pong.
//
// Same function as extend_attn_kernel (dkv_extend.cuh): new rows attend the past rows plus their own
// causal prefix (key j visible to new row i iff j <= seqlen_past + i; directkv/directkv_backend.py:887,
// csrc/directKV_kernel.cuh:654-678 in the reference).  That kernel runs QK^T -> softmax -> PV one after
// the other in four warps, so the tensor pipe waits for the softmax.  Here a CTA owns TWO 128-row query
// tiles and specialises its warps:
//
//   warp 0      TMA producer: both Q tiles once, then K(0), V(0), K(1), V(1), ... through a ring of 32 KB slots
//   warps 1, 2  MMA issuers (one thread each): S_g = Q_g K^T for tile g = 0 / 1
//   warps 3, 12 MMA issuers (one thread each): O_g += P_g V for tile g = 0 / 1
//   warps 4-7   softmax of tile 0 (thread = query row = TMEM lane)
//   warps 8-11  softmax of tile 1
//
// The keys of a 128-row K/V tile are processed as two half-tiles of 64, each with its own S buffer in TMEM
// in TMEM, so the issuer runs two half-tiles ahead of a group's softmax
// (S(t+2) is being multiplied while S(t) is exponentiated) and P V(t) overlaps the sweep of t+1; the two
// groups fill each other's gaps.  P never touches shared memory: the bf16 probabilities are stored back
// over the S buffer they came from (two per 32-bit column) and the second product reads its A operand
// from tensor memory, which leaves room for a five-slot K/V ring.  O stays in TMEM: the P V product accumulates into it, and a row's
// reference maximum is only moved (O and l rescaled through tcgen05.ld/st) when the true maximum grew by
// more than 2^8, so most half-tiles never touch O outside the tensor core.  Probabilities are therefore at
// most 256; sums stay fp32 and the final O / l is exact in the same sense as before.
//
// TMEM columns: S_0 [0,64) [64,128)   S_1 [128,192) [192,256)   O_0 [256,384)   O_1 [384,512).
#pragma once

#include <type_traits>

#include "dkv_extend.cuh"


namespace dkv {

constexpr int kPpSlots = 5;                                   // ring of [128 x 128] bf16 tiles: K and V alternate
constexpr int kPpThreads = 416;                               // 13 warps: producer, 4 issuers, 2 x 4 softmax
constexpr int kPpSmem = 2 * kExtTileBytes /*Q0,Q1*/ + kPpSlots * kExtTileBytes + 256 + 1024;
constexpr float kPpRescaleStep = 8.f;                         // log2 units the maximum may lag behind where it is taken
constexpr float kPpOverflowLog2 = 40.f;                       // a probability above 2^40 sends a half-tile back for its maximum
constexpr float kPpOverflowSum = 1099511627776.f;             // 2^40: the same test on the row sum of a half-tile
constexpr int kPpHalf = 64;                                   // keys per half-tile
constexpr int kPpPolyMask = 6;                 // pairs i with (i & mask) == mask go to the FMA pipe: 6 = every fourth (measured best), 2 = every second, 0x40 = none

struct PpCtrl {
    uint64_t bar_q;
    uint64_t full[kPpSlots];
    uint64_t empty[kPpSlots];
    uint64_t bar_s[2][2];     // [g][buf] S_g(t) complete, buf = t & 1
    uint64_t bar_p[2][2];     // [g][buf] P_g(t) stored, S buffer consumed, O_g rescaled: one arrival per softmax warp
    uint64_t bar_o[2][2];     // [g][buf] O_g += P_g(t) V complete
    uint32_t tmem;
    volatile int abort;
};

__global__ void __launch_bounds__(kPpThreads, 1)
extend_attn_pp_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                      const __grid_constant__ CUtensorMap tmV, const ExtendParams p) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* sQ = smem;                                       // tile g at + g * 32 KB
    uint8_t* sRing = sQ + 2 * kExtTileBytes;
    PpCtrl* ctl = reinterpret_cast<PpCtrl*>(sRing + kPpSlots * kExtTileBytes);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int G = p.G, TQ = kExtTile / G;
    const int h = blockIdx.x / p.nsub, sub = blockIdx.x % p.nsub;
    const int qhead0 = h * p.g_total + sub * G;
    int qt, s_new, past, q_row0, row_slot0;
    if (p.items != nullptr) {                                 // ragged batch: the host sorted the work list
        const int2 it = p.items[blockIdx.y];
        qt = it.y;
        s_new = p.r_s_new[it.x];
        past = p.r_past[it.x];
        q_row0 = p.r_q_row0[it.x];
        row_slot0 = p.r_slot0[it.x];
    } else {
        const int b = blockIdx.z;
        qt = static_cast<int>(gridDim.y) - 1 - static_cast<int>(blockIdx.y);   // longest (latest) tiles first
        s_new = p.S_new;
        past = p.n_past_blocks ? p.n_past_blocks[0] * 64 : p.seqlen_past;
        q_row0 = b * p.S_new;
        row_slot0 = static_cast<int>(static_cast<long long>(p.vrow ? p.vrow[b] : b) * p.row_stride);
    }
    const int q0 = qt * 2 * TQ;                               // first new token of tile 0; tile 1 starts at q0 + TQ
    const int s_total = past + s_new;
    int n_half[2];                                            // half-tiles of 64 keys each group walks
#pragma unroll
    for (int g = 0; g < 2; ++g) {
        int kv_end = p.is_causal ? past + q0 + (g + 1) * TQ : s_total;
        if (kv_end > s_total) kv_end = s_total;
        n_half[g] = (kv_end + kPpHalf - 1) / kPpHalf;         // n_half[1] >= n_half[0] >= 1 ...
        if (q0 + g * TQ >= s_new) n_half[g] = 0;              // ... unless tile 1 lies past the last new row: it does nothing
    }
    const int n_max = ((n_half[1] > n_half[0] ? n_half[1] : n_half[0]) + 1) >> 1;   // K/V tiles to load

    if (tid == 0) {
        mbar_init(&ctl->bar_q, 1);
        for (int s = 0; s < kPpSlots; ++s) {
            mbar_init(&ctl->full[s], 1);
            mbar_init(&ctl->empty[s], 2);                     // one arrival per query tile (the issuer that reads the slot)
        }
        for (int g = 0; g < 2; ++g)
            for (int bf = 0; bf < 2; ++bf) {
                mbar_init(&ctl->bar_s[g][bf], 1);
                mbar_init(&ctl->bar_p[g][bf], 4);
                mbar_init(&ctl->bar_o[g][bf], 1);
            }
        ctl->abort = 0;
        fence_mbar_init();
        fence_proxy_async_smem();
        tma_prefetch_desc(&tmQ);
        tma_prefetch_desc(&tmK);
        tma_prefetch_desc(&tmV);
    }
    if (warp == 1) {
        tmem_alloc(&ctl->tmem, 512);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = ctl->tmem;

    if (warp == 0) {
        // ------------------------------------------------ TMA producer ------------------------------------------------
        if (lane == 0) {
            mbar_arrive_expect_tx(&ctl->bar_q, 2 * kExtTileBytes);
#pragma unroll
            for (int g = 0; g < 2; ++g) {
                // Rows r = t * G + head come as a (d, head, token) box: G heads of TQ tokens.
                tma_load_3d(sQ + g * kExtTileBytes, &tmQ, &ctl->bar_q, 0, qhead0, q_row0 + q0 + g * TQ);
                tma_load_3d(sQ + g * kExtTileBytes + kExtHalfBytes, &tmQ, &ctl->bar_q, 64, qhead0, q_row0 + q0 + g * TQ);
            }
            for (int q = 0; q < 2 * n_max; ++q) {             // q even: K(q/2), odd: V(q/2)
                const int s = q % kPpSlots;
                if (q >= kPpSlots && !mbar_wait_bounded(&ctl->empty[s], ((q / kPpSlots) - 1) & 1)) {
                    atomicOr(p.status, kStatusWaitTimeout | kStatusInExtend);
                    ctl->abort = 1;
                    break;
                }
                if (ctl->abort) break;
                uint8_t* dst = sRing + s * kExtTileBytes;
                const CUtensorMap* tm = (q & 1) ? &tmV : &tmK;
                const int slot = row_slot0 + (q >> 1) * kExtTile;
                mbar_arrive_expect_tx(&ctl->full[s], kExtTileBytes);
                tma_load_3d(dst, tm, &ctl->full[s], 0, h, slot);
                tma_load_3d(dst + kExtHalfBytes, tm, &ctl->full[s], 64, h, slot);
                // A slot is released by one arrival per query tile.  A tile that walks fewer keys than the other (or
                // none: tile 1 past the last new row) never reads this K/V tile, and the producer - the one thread that
                // follows every phase of the slot in order - arrives in its place.  (The tile's own issuer must not do
                // it from a loop that runs ahead of the loads: it sees only every other phase of a slot, K and V
                // alternate there, and a parity wait on a barrier that is a phase behind returns at once.)
#pragma unroll
                for (int g = 0; g < 2; ++g)
                    if ((q >> 1) >= ((n_half[g] + 1) >> 1)) mbar_arrive(&ctl->empty[s]);
            }
        }
        __syncwarp();
    } else if (warp == 1 || warp == 2) {
        // ------------------------------------------------ MMA issuers: S = Q K^T ------------------------------------------------
        // One thread per query tile and product (warps 1, 2: S of tile 0 / 1; warps 3, 12: P V of tile 0 / 1).  A
        // tcgen05.mma blocks its thread while the pipe is busy and every commit and wait costs it another hundred
        // cycles or so, so the fewer steps a thread has per half-tile, the less the pipe idles.  Descriptors are built
        // once; inside the loops only constants are added to them.
        if (lane == 0) {
            const int g = warp - 1;
            const int n_g = n_half[g];
            constexpr uint32_t idesc_qk = umma_idesc_bf16_f32(kExtTile, kPpHalf);
            const uint64_t q_desc = umma_desc_k_sw128(smem_u32(sQ + g * kExtTileBytes));
            const uint64_t k_desc0 = umma_desc_k_sw128(smem_u32(sRing));
            const uint32_t tS = tmem_base + g * 128;
            bool ok = mbar_wait_bounded(&ctl->bar_q, 0);
            for (int t = 0; ok && t < n_g; ++t) {
                const int q = 2 * (t >> 1), slot = q % kPpSlots;
                // Buffer t & 1 holds P(t - 2) until the product that reads it is complete (another thread issues it).
                if (t >= 2) ok = mbar_wait_bounded(&ctl->bar_o[g][t & 1], ((t - 2) >> 1) & 1) && !ctl->abort;
                if (ok && !(t & 1)) ok = mbar_wait_bounded(&ctl->full[slot], (q / kPpSlots) & 1);
                if (!ok) break;
                tc_fence_after_sync();
                const uint64_t kd = k_desc0 + static_cast<uint64_t>((slot * kExtTileBytes + (t & 1) * kPpHalf * 128) >> 4);
                const uint32_t d = tS + (t & 1) * kPpHalf;
#pragma unroll
                for (int k = 0; k < 8; ++k) {
                    constexpr int unit = 16;                  // descriptor addresses count 16-byte units
                    const uint64_t off = static_cast<uint64_t>(((k >> 2) * kExtHalfBytes + (k & 3) * 32) / unit);
                    umma_bf16_ss(d, q_desc + off, kd + off, idesc_qk, k > 0 ? 1u : 0u);
                }
                umma_commit(&ctl->bar_s[g][t & 1]);
                if ((t & 1) || t == n_g - 1) umma_commit(&ctl->empty[slot]);   // this tile's last read of K(t >> 1)
            }
            if (!ok) {
                atomicOr(p.status, kStatusWaitTimeout | kStatusInExtend);
                ctl->abort = 1;
            }
        }
        __syncwarp();
    } else if (warp == 3 || warp == 12) {
        // ------------------------------------------------ MMA issuers: O += P V ------------------------------------------------
        if (lane == 0) {
            const int g = warp == 3 ? 0 : 1;
            const int n_g = n_half[g];
            constexpr uint32_t idesc_pv = umma_idesc_bf16_f32(kExtTile, kExtTile) | (1u << 16);   // B (V) is MN-major
            const uint64_t v_desc0 = umma_desc_mn_sw128(smem_u32(sRing), kExtHalfBytes);
            const uint32_t tS = tmem_base + g * 128, tO = tmem_base + 256 + g * 128;
            bool ok = true;
            for (int t = 0; ok && t < n_g; ++t) {
                const int q = 2 * (t >> 1) + 1, slot = q % kPpSlots;
                ok = mbar_wait_bounded(&ctl->bar_p[g][t & 1], (t >> 1) & 1) && !ctl->abort;
                if (ok && !(t & 1)) ok = mbar_wait_bounded(&ctl->full[slot], (q / kPpSlots) & 1);
                if (!ok) break;
                tc_fence_after_sync();
                const uint64_t vd = v_desc0 + static_cast<uint64_t>((slot * kExtTileBytes + (t & 1) * kPpHalf * 128) >> 4);
                const uint32_t pa = tS + (t & 1) * kPpHalf;   // P lies over the S buffer it came from
#pragma unroll
                for (int k = 0; k < 4; ++k)                   // 16 keys per step = 8 packed columns of P, 16 rows of V
                    umma_bf16_ts(tO, pa + k * 8, vd + static_cast<uint64_t>((k * 16 * 128) >> 4), idesc_pv, (t > 0 || k > 0) ? 1u : 0u);
                umma_commit(&ctl->bar_o[g][t & 1]);
                if ((t & 1) || t == n_g - 1) umma_commit(&ctl->empty[slot]);
            }
            if (!ok) {
                atomicOr(p.status, kStatusWaitTimeout | kStatusInExtend);
                ctl->abort = 1;
            }
        }
        __syncwarp();
    }

    if (warp >= 4 && warp < 12) {
        // ------------------------------------------------ softmax groups ------------------------------------------------
        const int g = (warp - 4) >> 2;                        // query tile of this warp
        const int row = ((warp & 3) << 5) + lane;             // TMEM lane == query row of the tile
        const int my_tok = q0 + g * TQ + row / G;             // new-token index of the row
        const int my_limit = p.is_causal ? past + my_tok : s_total - 1;           // last visible key
        const int first_limit = p.is_causal ? past + q0 + g * TQ : s_total - 1;   // smallest limit in the tile
        const uint32_t lane_sel = static_cast<uint32_t>((warp & 3) * 32) << 16;
        const uint32_t tS = tmem_base + lane_sel + g * 128;
        const uint32_t tO = tmem_base + lane_sel + 256 + g * 128;
        const int n_g = n_half[g];
        float m_used = -INFINITY, l = 0.f;
        bool ok = true;

        for (int t = 0; t < n_g; ++t) {
            const int bf = t & 1;
            // S(t) complete; the product that wrote it was issued after P V(t - 2) had completed and read the buffer.
            ok = __all_sync(0xffffffffu, mbar_wait_bounded(&ctl->bar_s[g][bf], (t >> 1) & 1) && !ctl->abort);
            if (!ok) break;
            tc_fence_after_sync();
            const int col0 = t * kPpHalf;
            const uint32_t tSb = tS + bf * kPpHalf;
            // Warp-uniform: only half-tiles on the diagonal (or holding the end of the request) need the comparison.
            const bool masked = (col0 + kPpHalf - 1 > first_limit) || !(p.scale_log2 > 0.f);
            uint32_t r0[32], r1[32], pk[32];                  // the row's 64 scores stay in registers
            float psum;
            // Most half-tiles take no row maximum at all: probabilities are formed against the reference the row
            // already has, and only if one of them would come out above 2^kPpOverflowLog2 (seen in the sum, and for
            // the pairs on the FMA pipe in their arguments) is the half-tile done again with its maximum taken and
            // the reference moved.  Floating point keeps the relative precision of P, l and O whatever the offset.
            // Returns whether the half-tile has to be done again with its maximum taken (never when it was).
            auto sweep = [&](auto with_max_tag) -> bool {
                constexpr bool with_max = decltype(with_max_tag)::value;
                tmem_ld_32x32(tSb, r0);
                tmem_ld_32x32(tSb + 32, r1);
                tmem_ld_wait();
                if constexpr (with_max) {
                    float m_tile = -INFINITY;
                    if (masked) {
#pragma unroll
                        for (int i = 0; i < 32; ++i) {
                            if (col0 + i <= my_limit) m_tile = fmaxf(m_tile, __uint_as_float(r0[i]) * p.scale_log2);
                            if (col0 + 32 + i <= my_limit) m_tile = fmaxf(m_tile, __uint_as_float(r1[i]) * p.scale_log2);
                        }
                    } else {
                        float a0 = -INFINITY, a1 = -INFINITY, a2 = -INFINITY, a3 = -INFINITY;     // four short chains
#pragma unroll
                        for (int i = 0; i < 16; i += 2) {
                            a0 = fmax3(a0, __uint_as_float(r0[i]), __uint_as_float(r0[i + 1]));
                            a1 = fmax3(a1, __uint_as_float(r0[16 + i]), __uint_as_float(r0[17 + i]));
                            a2 = fmax3(a2, __uint_as_float(r1[i]), __uint_as_float(r1[i + 1]));
                            a3 = fmax3(a3, __uint_as_float(r1[16 + i]), __uint_as_float(r1[17 + i]));
                        }
                        a0 = fmaxf(a0, a2);
                        a1 = fmaxf(a1, a3);
                        m_tile = fmaxf(a0, a1) * p.scale_log2;            // scale_log2 > 0 on this path
                    }
                    // Move the reference only when the true maximum is more than the step above it (warp-uniform):
                    // then O and l are rescaled; otherwise probabilities are formed against the old reference.
                    const bool grow = (m_tile > m_used + kPpRescaleStep) || (m_used == -INFINITY);
                    if (__any_sync(0xffffffffu, grow)) {
                        float m_to = fmaxf(m_used, m_tile);
                        if (m_to == -INFINITY) m_to = 0.f;
                        const float alpha = exp2f(m_used - m_to);             // 0 on the first half-tile
                        l *= alpha;
                        m_used = m_to;
                        if (t > 0) {
                            // O must be at rest: P V(t - 1) is the last product issued for this tile.
                            ok = __all_sync(0xffffffffu, mbar_wait_bounded(&ctl->bar_o[g][(t - 1) & 1], ((t - 1) >> 1) & 1) && !ctl->abort);
                            if (!ok) return false;
                            tc_fence_after_sync();
#pragma unroll 1
                            for (int c = 0; c < 4; ++c) {
                                uint32_t r[32];
                                tmem_ld_32x32(tO + c * 32, r);
                                tmem_ld_wait();
#pragma unroll
                                for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
                                tmem_st_32x32(tO + c * 32, r);
                            }
                            tmem_st_wait();
                        }
                    }
                }
                // Probabilities, packed two bf16 per 32-bit column, go back into the first 32 columns of the S buffer.
                // In place and in phases (scale and shift, exponentials, mask, sums and packing), so that each phase is
                // a run of independent instructions on one pipe.
                const float neg_m = -m_used;
                const uint64_t sc2 = f32x2(p.scale_log2, p.scale_log2), nm2 = f32x2(neg_m, neg_m);
                float* x0 = reinterpret_cast<float*>(r0);
                float* x1 = reinterpret_cast<float*>(r1);
#pragma unroll
                for (int i = 0; i < 32; i += 2) {
                    f32x2_split(fma_f32x2(f32x2(x0[i], x0[i + 1]), sc2, nm2), x0[i], x0[i + 1]);
                    f32x2_split(fma_f32x2(f32x2(x1[i], x1[i + 1]), sc2, nm2), x1[i], x1[i + 1]);
                }
                float big = -INFINITY;                        // largest argument among the pairs of the FMA pipe
                if constexpr (!with_max) {
#pragma unroll
                    for (int i = 0; i < 32; i += 2)
                        if ((i & kPpPolyMask) == kPpPolyMask) {
                            big = fmax3(big, x0[i], x0[i + 1]);
                            big = fmax3(big, x1[i], x1[i + 1]);
                        }
                }
#pragma unroll
                for (int i = 0; i < 32; i += 2) {
                    if ((i & kPpPolyMask) == kPpPolyMask) {       // this pair on the FMA pipe
                        f32x2_split(ex2_poly_f32x2(f32x2(x0[i], x0[i + 1])), x0[i], x0[i + 1]);
                        f32x2_split(ex2_poly_f32x2(f32x2(x1[i], x1[i + 1])), x1[i], x1[i + 1]);
                    } else {
                        x0[i] = ex2_approx(x0[i]);
                        x0[i + 1] = ex2_approx(x0[i + 1]);
                        x1[i] = ex2_approx(x1[i]);
                        x1[i + 1] = ex2_approx(x1[i + 1]);
                    }
                }
                if (masked) {
#pragma unroll
                    for (int i = 0; i < 32; ++i) {
                        if (col0 + i > my_limit) x0[i] = 0.f;
                        if (col0 + 32 + i > my_limit) x1[i] = 0.f;
                    }
                }
                uint64_t sa = f32x2(0.f, 0.f), sb = sa;
#pragma unroll
                for (int i = 0; i < 32; i += 2) {
                    sa = add_f32x2(sa, f32x2(x0[i], x0[i + 1]));
                    sb = add_f32x2(sb, f32x2(x1[i], x1[i + 1]));
                    pk[i >> 1] = pack_bf16x2(x0[i], x0[i + 1]);
                    pk[16 + (i >> 1)] = pack_bf16x2(x1[i], x1[i + 1]);
                }
                float s4[4];
                f32x2_split(sa, s4[0], s4[1]);
                f32x2_split(sb, s4[2], s4[3]);
                psum = (s4[0] + s4[1]) + (s4[2] + s4[3]);
                if constexpr (with_max) return false;
                // NaN and infinity fail the first comparison too.
                const bool over = !(psum < kPpOverflowSum) || big > kPpOverflowLog2;
                return __any_sync(0xffffffffu, over);
            };
            if ((t == 0) || masked) {
                sweep(std::true_type{});
            } else if (sweep(std::false_type{})) {
                sweep(std::true_type{});                      // S(t) is still in tensor memory: once more, with its maximum
            }
            if (!ok) break;
            tmem_st_32x32(tSb, pk);
            tmem_st_wait();
            l += psum;
            // Rows of the last tile past the request's last token may hold anything: V must be finite there
            // because P (zero) still multiplies it.  Done with the tile's first half; both groups write the same zeros.
            const int tile_valid = s_total - (t >> 1) * kExtTile;
            if (bf == 0 && tile_valid < kExtTile) {
                const int q = 2 * (t >> 1) + 1;
                uint8_t* sV = sRing + (q % kPpSlots) * kExtTileBytes;
                ok = __all_sync(0xffffffffu, mbar_wait_bounded(&ctl->full[q % kPpSlots], (q / kPpSlots) & 1) && !ctl->abort);
                if (!ok) break;
                for (int idx = row; idx < (kExtTile - tile_valid) * 16; idx += 128) {
                    const int r = tile_valid + idx / 16, c = idx % 16;
                    *reinterpret_cast<uint4*>(sV + (c >> 3) * kExtHalfBytes + r * 128 + ((c & 7) << 4)) = make_uint4(0, 0, 0, 0);
                }
                fence_proxy_async_smem();
            }
            // One arrival per warp: 32 lanes arriving on the same mbarrier would serialise.
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(&ctl->bar_p[g][bf]);
        }

        if (n_g == 0) {
            ok = true;           // an empty tile: nothing to wait for, nothing to store
        } else if (ok) {
            // The last two products (one per P buffer) end the accumulation.
            if (n_g >= 2)
                ok = __all_sync(0xffffffffu, mbar_wait_bounded(&ctl->bar_o[g][(n_g - 2) & 1], ((n_g - 2) >> 1) & 1) && !ctl->abort);
            if (ok) ok = __all_sync(0xffffffffu, mbar_wait_bounded(&ctl->bar_o[g][(n_g - 1) & 1], ((n_g - 1) >> 1) & 1) && !ctl->abort);
            tc_fence_after_sync();
        }
        if (!ok) {
            if (lane == 0) atomicOr(p.status, kStatusWaitTimeout | kStatusInExtend);
            ctl->abort = 1;
        } else if (n_g > 0) {
            const float inv = l > 0.f ? 1.f / l : 0.f;
            const bool store = my_tok < s_new;
            __nv_bfloat16* dst = p.out + ((static_cast<long long>(q_row0) + (store ? my_tok : 0)) * p.nh_q + qhead0 + row % G) * 128;
#pragma unroll 1
            for (int c = 0; c < 4; ++c) {
                uint32_t r[32];
                tmem_ld_32x32(tO + c * 32, r);
                tmem_ld_wait();
                if (store) {
#pragma unroll
                    for (int q8 = 0; q8 < 4; ++q8) {
                        uint4 w;
                        w.x = pack_bf16x2(__uint_as_float(r[q8 * 8 + 0]) * inv, __uint_as_float(r[q8 * 8 + 1]) * inv);
                        w.y = pack_bf16x2(__uint_as_float(r[q8 * 8 + 2]) * inv, __uint_as_float(r[q8 * 8 + 3]) * inv);
                        w.z = pack_bf16x2(__uint_as_float(r[q8 * 8 + 4]) * inv, __uint_as_float(r[q8 * 8 + 5]) * inv);
                        w.w = pack_bf16x2(__uint_as_float(r[q8 * 8 + 6]) * inv, __uint_as_float(r[q8 * 8 + 7]) * inv);
                        *reinterpret_cast<uint4*>(dst + c * 32 + q8 * 8) = w;
                    }
                }
            }
        }
    }

    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem_base, 512);
}

}  // namespace dkv
