// Extend / chunked-prefill attention, two query tiles per CTA in ping-pong.
//
// Same function as extend_attn_kernel (dkv_extend.cuh): new rows attend the past rows plus their own
// causal prefix (key j visible to new row i iff j <= seqlen_past + i; directkv/directkv_backend.py:887,
// csrc/directKV_kernel.cuh:654-678 in the reference).  That kernel runs QK^T -> softmax -> PV one after
// the other in four warps, so the tensor pipe waits for the softmax.  Here a CTA owns TWO 128-row query
// tiles and specialises its warps:
//
//   warp 0      TMA producer: both Q tiles once, then K(0), V(0), K(1), V(1), ... through a ring of 32 KB slots
//   warp 1      MMA issuer (one thread): S_g = Q_g K^T and O_g += P_g V for g = 0, 1
//   warps 4-7   softmax of tile 0 (thread = query row = TMEM lane)
//   warps 8-11  softmax of tile 1
//
// While one group exponentiates, the tensor core works for the other.  O stays in TMEM: the P V product
// accumulates into it, and a row's running maximum is only moved (O and l rescaled through tcgen05.ld/st)
// when it grew by more than 2^8, so most tiles never touch O outside the tensor core.  Probabilities are
// therefore at most 256; sums stay fp32 and the final O / l is exact in the same sense as before.
//
// TMEM columns: S_0 [0,128)  S_1 [128,256)  O_0 [256,384)  O_1 [384,512).
#pragma once

#include "dkv_extend.cuh"

namespace dkv {

constexpr int kPpSlots = 3;                                   // ring of [128 x 128] bf16 tiles: K and V alternate
constexpr int kPpThreads = 384;
constexpr int kPpSmem = 2 * kExtTileBytes /*Q0,Q1*/ + 2 * kExtTileBytes /*P0,P1*/ + kPpSlots * kExtTileBytes + 256 + 1024;
constexpr float kPpRescaleStep = 8.f;                         // log2 units the maximum may lag behind

struct PpCtrl {
    uint64_t bar_q;
    uint64_t full[kPpSlots];
    uint64_t empty[kPpSlots];
    uint64_t bar_s[2];        // S_g(j) complete
    uint64_t bar_p[2];        // P_g(j) stored, S_g consumed, O_g rescaled: 128 arrivals
    uint64_t bar_o[2];        // O_g += P_g V(j) complete
    uint32_t tmem;
    volatile int abort;
};

__global__ void __launch_bounds__(kPpThreads, 1)
extend_attn_pp_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                      const __grid_constant__ CUtensorMap tmV, const ExtendParams p) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* sQ = smem;                                       // tile g at + g * 32 KB
    uint8_t* sP = sQ + 2 * kExtTileBytes;
    uint8_t* sRing = sP + 2 * kExtTileBytes;
    PpCtrl* ctl = reinterpret_cast<PpCtrl*>(sRing + kPpSlots * kExtTileBytes);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int G = p.G, TQ = kExtTile / G;
    const int qt = static_cast<int>(gridDim.x) - 1 - static_cast<int>(blockIdx.x);   // longest (latest) tiles first
    const int b = blockIdx.z;
    const int h = blockIdx.y / p.nsub, sub = blockIdx.y % p.nsub;
    const int qhead0 = h * p.g_total + sub * G;
    const int past = p.n_past_blocks ? p.n_past_blocks[0] * 64 : p.seqlen_past;
    const int q0 = qt * 2 * TQ;                               // first new token of tile 0; tile 1 starts at q0 + TQ
    const int row_slot0 = static_cast<int>(static_cast<long long>(p.vrow ? p.vrow[b] : b) * p.row_stride);
    const int s_total = past + p.S_new;
    int n_tiles[2];
#pragma unroll
    for (int g = 0; g < 2; ++g) {
        int kv_end = p.is_causal ? past + q0 + (g + 1) * TQ : s_total;
        if (kv_end > s_total) kv_end = s_total;
        n_tiles[g] = (kv_end + kExtTile - 1) / kExtTile;      // n_tiles[1] >= n_tiles[0] >= 1
    }
    const int n_max = n_tiles[1];

    if (tid == 0) {
        mbar_init(&ctl->bar_q, 1);
        for (int s = 0; s < kPpSlots; ++s) {
            mbar_init(&ctl->full[s], 1);
            mbar_init(&ctl->empty[s], 1);
        }
        for (int g = 0; g < 2; ++g) {
            mbar_init(&ctl->bar_s[g], 1);
            mbar_init(&ctl->bar_p[g], 128);
            mbar_init(&ctl->bar_o[g], 1);
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
                tma_load_3d(sQ + g * kExtTileBytes, &tmQ, &ctl->bar_q, 0, qhead0, b * p.S_new + q0 + g * TQ);
                tma_load_3d(sQ + g * kExtTileBytes + kExtHalfBytes, &tmQ, &ctl->bar_q, 64, qhead0, b * p.S_new + q0 + g * TQ);
            }
            for (int q = 0; q < 2 * n_max; ++q) {             // q even: K(q/2), odd: V(q/2)
                const int s = q % kPpSlots;
                if (q >= kPpSlots && !mbar_wait_bounded(&ctl->empty[s], ((q / kPpSlots) - 1) & 1)) {
                    atomicOr(p.status, kStatusWaitTimeout);
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
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ------------------------------------------------ MMA issuer ------------------------------------------------
        if (lane == 0) {
            constexpr uint32_t idesc_qk = umma_idesc_bf16_f32(kExtTile, kExtTile);
            constexpr uint32_t idesc_pv = umma_idesc_bf16_f32(kExtTile, kExtTile) | (1u << 16);   // B (V) is MN-major
            bool ok = mbar_wait_bounded(&ctl->bar_q, 0);
            int ring_ready = -1;                              // highest ring sequence number known to have landed
            auto wait_ring = [&](int q) {
                while (ok && ring_ready < q) {
                    const int nq = ring_ready + 1;
                    ok = mbar_wait_bounded(&ctl->full[nq % kPpSlots], (nq / kPpSlots) & 1);
                    ring_ready = nq;
                }
            };
            auto issue_qk = [&](int g, int j) {               // S_g = Q_g K(j)^T
                const uint32_t qa = smem_u32(sQ + g * kExtTileBytes), ka = smem_u32(sRing + ((2 * j) % kPpSlots) * kExtTileBytes);
#pragma unroll
                for (int k = 0; k < 8; ++k) {
                    const uint32_t off = (k >> 2) * kExtHalfBytes + (k & 3) * 32;
                    umma_bf16_ss(tmem_base + g * 128, umma_desc_k_sw128(qa + off), umma_desc_k_sw128(ka + off), idesc_qk,
                                 k > 0 ? 1u : 0u);
                }
                umma_commit(&ctl->bar_s[g]);
                if (g == 1) umma_commit(&ctl->empty[(2 * j) % kPpSlots]);       // tile 1 is the last reader of K(j)
            };
            auto issue_pv = [&](int g, int j) {               // O_g (+)= P_g V(j)
                const uint32_t pa = smem_u32(sP + g * kExtTileBytes), va = smem_u32(sRing + ((2 * j + 1) % kPpSlots) * kExtTileBytes);
#pragma unroll
                for (int k = 0; k < 8; ++k) {
                    const uint32_t aoff = (k >> 2) * kExtHalfBytes + (k & 3) * 32;   // 16 keys along K of P
                    const uint32_t boff = k * 16 * 128;                               // 16 key rows of V
                    umma_bf16_ss(tmem_base + 256 + g * 128, umma_desc_k_sw128(pa + aoff),
                                 umma_desc_mn_sw128(va + boff, kExtHalfBytes), idesc_pv, (j > 0 || k > 0) ? 1u : 0u);
                }
                umma_commit(&ctl->bar_o[g]);
                if (g == 1) umma_commit(&ctl->empty[(2 * j + 1) % kPpSlots]);
            };
            wait_ring(0);
            if (ok) {
                tc_fence_after_sync();
                issue_qk(0, 0);
                issue_qk(1, 0);
            }
            for (int j = 0; ok && j < n_max; ++j) {
                for (int g = 0; ok && g < 2; ++g) {
                    if (j >= n_tiles[g]) continue;
                    ok = mbar_wait_bounded(&ctl->bar_p[g], j & 1) && !ctl->abort;
                    if (!ok) break;
                    tc_fence_after_sync();
                    if (j + 1 < n_tiles[g]) {
                        wait_ring(2 * (j + 1));
                        if (!ok) break;
                        tc_fence_after_sync();
                        issue_qk(g, j + 1);
                    }
                    wait_ring(2 * j + 1);
                    if (!ok) break;
                    tc_fence_after_sync();
                    issue_pv(g, j);
                }
            }
            if (!ok) {
                atomicOr(p.status, kStatusWaitTimeout);
                ctl->abort = 1;
            }
        }
        __syncwarp();
    }

    if (warp >= 4) {
        // ------------------------------------------------ softmax groups ------------------------------------------------
        const int g = (warp - 4) >> 2;                        // query tile of this warp
        const int row = ((warp & 3) << 5) + lane;             // TMEM lane == query row of the tile
        const int my_tok = q0 + g * TQ + row / G;             // new-token index of the row
        const int my_limit = p.is_causal ? past + my_tok : s_total - 1;           // last visible key
        const int first_limit = p.is_causal ? past + q0 + g * TQ : s_total - 1;   // smallest limit in the tile
        const uint32_t lane_sel = static_cast<uint32_t>((warp & 3) * 32) << 16;
        const uint32_t tS = tmem_base + lane_sel + g * 128;
        const uint32_t tO = tmem_base + lane_sel + 256 + g * 128;
        uint8_t* sPg = sP + g * kExtTileBytes;
        const int n_g = n_tiles[g];
        float m_used = -INFINITY, l = 0.f;
        bool ok = true;

        for (int j = 0; j < n_g; ++j) {
            ok = __all_sync(0xffffffffu, mbar_wait_bounded(&ctl->bar_s[g], j & 1) && !ctl->abort);
            if (!ok) break;
            tc_fence_after_sync();
            const int col0 = j * kExtTile;
            // Warp-uniform: only tiles on the diagonal (or holding the end of the request) need the comparison.
            const bool masked = (col0 + kExtTile - 1 > first_limit) || !(p.scale_log2 > 0.f);
            // The previous P V of this tile must be done before P is overwritten or O is touched.
            if (j > 0) {
                ok = __all_sync(0xffffffffu, mbar_wait_bounded(&ctl->bar_o[g], (j - 1) & 1) && !ctl->abort);
                if (!ok) break;
                tc_fence_after_sync();
            }
            // One pass over S in the common case: probabilities are formed against the maximum in use while
            // the tile's own maximum is tracked; only when that one is more than the step above (or on the
            // first tile) is the maximum moved, O and l rescaled, and the pass repeated.
            float psum = 0.f, m_tile = -INFINITY;
            auto sweep = [&](const float neg_m, const bool track) {
                psum = 0.f;
#pragma unroll 1
                for (int c = 0; c < 4; ++c) {
                    uint32_t r[32];
                    tmem_ld_32x32(tS + c * 32, r);
                    tmem_ld_wait();
                    float pv[32];
                    if (masked) {
#pragma unroll
                        for (int i = 0; i < 32; ++i) {
                            const bool vis = col0 + c * 32 + i <= my_limit;
                            const float sc = __uint_as_float(r[i]) * p.scale_log2;
                            if (track && vis) m_tile = fmaxf(m_tile, sc);
                            pv[i] = vis ? ex2_approx(sc + neg_m) : 0.f;
                            psum += pv[i];
                        }
                    } else {
                        float raw = -INFINITY;
#pragma unroll
                        for (int i = 0; i < 32; ++i) {
                            if (track) raw = fmaxf(raw, __uint_as_float(r[i]));
                            pv[i] = ex2_approx(fmaf(__uint_as_float(r[i]), p.scale_log2, neg_m));
                            psum += pv[i];
                        }
                        if (track) m_tile = fmaxf(m_tile, raw * p.scale_log2);   // scale_log2 > 0 on this path
                    }
#pragma unroll
                    for (int q8 = 0; q8 < 4; ++q8) {
                        uint4 w;
                        w.x = pack_bf16x2(pv[q8 * 8 + 0], pv[q8 * 8 + 1]);
                        w.y = pack_bf16x2(pv[q8 * 8 + 2], pv[q8 * 8 + 3]);
                        w.z = pack_bf16x2(pv[q8 * 8 + 4], pv[q8 * 8 + 5]);
                        w.w = pack_bf16x2(pv[q8 * 8 + 6], pv[q8 * 8 + 7]);
                        const int c8 = c * 4 + q8;             // 16-byte chunk within the 128-key row
                        *reinterpret_cast<uint4*>(sPg + (c8 >> 3) * kExtHalfBytes + row * 128 + (((c8 & 7) ^ (row & 7)) << 4)) = w;
                    }
                }
            };
            if (j == 0) {
                // No maximum yet: a tracking-only sweep would waste the exponentials, so find the maximum first.
#pragma unroll 1
                for (int c = 0; c < 4; ++c) {
                    uint32_t r[32];
                    tmem_ld_32x32(tS + c * 32, r);
                    tmem_ld_wait();
#pragma unroll
                    for (int i = 0; i < 32; ++i)
                        if (!masked || col0 + c * 32 + i <= my_limit) m_tile = fmaxf(m_tile, __uint_as_float(r[i]) * p.scale_log2);
                }
            } else {
                sweep(-m_used, true);
            }
            const bool grow = (m_tile > m_used + kPpRescaleStep) || (m_used == -INFINITY);
            if (__any_sync(0xffffffffu, grow)) {                      // warp-uniform
                float m_to = fmaxf(m_used, m_tile);
                if (m_to == -INFINITY) m_to = 0.f;
                const float alpha = exp2f(m_used - m_to);             // 0 on the first tile
                l *= alpha;
                m_used = m_to;
                if (j > 0) {
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
                sweep(-m_used, false);
            }
            l += psum;
            // Rows of the last tile past the request's last token may hold anything: V must be finite there
            // because P (zero) still multiplies it.  Both groups write the same zeros.
            const int tile_valid = s_total - col0;
            if (tile_valid < kExtTile) {
                uint8_t* sV = sRing + ((2 * j + 1) % kPpSlots) * kExtTileBytes;
                ok = __all_sync(0xffffffffu, mbar_wait_bounded(&ctl->full[(2 * j + 1) % kPpSlots], ((2 * j + 1) / kPpSlots) & 1));
                if (!ok) break;
                for (int idx = row; idx < (kExtTile - tile_valid) * 16; idx += 128) {
                    const int r = tile_valid + idx / 16, c = idx % 16;
                    *reinterpret_cast<uint4*>(sV + (c >> 3) * kExtHalfBytes + r * 128 + ((c & 7) << 4)) = make_uint4(0, 0, 0, 0);
                }
            }
            fence_proxy_async_smem();
            tc_fence_before_sync();
            mbar_arrive(&ctl->bar_p[g]);
        }

        if (ok) {
            ok = __all_sync(0xffffffffu, mbar_wait_bounded(&ctl->bar_o[g], (n_g - 1) & 1) && !ctl->abort);
            tc_fence_after_sync();
        }
        if (!ok) {
            if (lane == 0) atomicOr(p.status, kStatusWaitTimeout);
            ctl->abort = 1;
        } else {
            const float inv = l > 0.f ? 1.f / l : 0.f;
            const bool store = my_tok < p.S_new;
            __nv_bfloat16* dst = p.out + ((static_cast<long long>(b) * p.S_new + (store ? my_tok : 0)) * p.nh_q + qhead0 + row % G) * 128;
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
