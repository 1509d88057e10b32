// Streaming split-KV decode attention for grouped queries (3..16 query heads per KV head).
//
// Same work decomposition, cursors, partial records and merge as dkv_attn.cuh; only the inner product
// differs.  With G query heads sharing a KV head the per-byte arithmetic (G FMAs per bf16 element) makes
// the CUDA-core kernel issue-bound at G = 4, so here the G query rows form the (zero-padded) 16-row M side
// of warp-level tensor-core products:
//
//   S[16 x 16 tokens] = Q[16 x 128] . K_tile^T      8 k-steps x 2 token halves  = 16 mma.m16n8k16
//   O[16 x 128]      += P[16 x 16]  . V_tile        16 head-dim slices          = 16 mma.m16n8k16
//
// K and V tiles come by TMA as two 64-column boxes with the 128-byte swizzle, which makes every ldmatrix
// (plain for K, transposed for V) conflict-free; the S accumulators are already laid out as the A operand
// of the second product, so probabilities go from registers to the tensor core without a shuffle.
// Scores, maxima and sums stay fp32; probabilities are rounded to bf16 for the second product.
//
// (tcgen05 is not used here on purpose: its smallest tile is 64 rows and its accumulator lives in TMEM
// behind a commit/wait round trip per tile; for 4..16 live rows per 16-token tile the warp-level
// instruction is the right size.)
#pragma once

#include "dkv_attn.cuh"

namespace dkv {

constexpr int kMmaHalfBytes = kTileTokens * 128;   // one [16 tokens x 64 bf16] swizzled block: 2 KB

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr));
}

__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr));
}

// D (fp32) += A (bf16, 16x16 row-major fragments) * B (bf16, 16x8 column fragments)
__device__ __forceinline__ void mma_bf16_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
        "{%0, %1, %2, %3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// Byte offset of 16-byte chunk `c16` (0..15 over the 256-byte row) of token row `t` inside a K or V tile that
// was loaded as two 128-byte-swizzled 64-column boxes.
__device__ __forceinline__ uint32_t sw_tile_off(int t, int c16) {
    return static_cast<uint32_t>((c16 >> 3) * kMmaHalfBytes + t * 128 + (((c16 & 7) ^ (t & 7)) << 4));
}

// Lane 0 only: TMA copies of one tile (K low/high columns, V low/high columns) into a stage laid out
// [K lo | K hi | V lo | V hi], 2 KB each.
__device__ __forceinline__ void issue_tile_sw(const AttnParams& p, const CUtensorMap* tmK, const CUtensorMap* tmV,
                                              const TileCursor& c, uint8_t* stage, uint64_t* bar) {
    const int h = c.hs / p.nsub;
    const int tok0 = c.tile * kTileTokens;
    const int row = p.row_map ? p.row_map[c.b] : c.b;
    auto four = [&](int dst_row, int slot) {
        uint8_t* d = stage + dst_row * 128;
        tma_load_3d(d, tmK, bar, 0, h, slot);
        tma_load_3d(d + kMmaHalfBytes, tmK, bar, 64, h, slot);
        tma_load_3d(d + 2 * kMmaHalfBytes, tmV, bar, 0, h, slot);
        tma_load_3d(d + 3 * kMmaHalfBytes, tmV, bar, 64, h, slot);
    };
    if (p.page_table == nullptr) {
        mbar_arrive_expect_tx(bar, kStageBytes);
        four(0, static_cast<int>(static_cast<long long>(row) * p.row_stride + tok0));
    } else if (p.page_size >= kTileTokens) {
        const int page = page_at(p, row, tok0 >> p.page_shift);
        mbar_arrive_expect_tx(bar, kStageBytes);
        four(0, static_cast<int>((static_cast<long long>(page) << p.page_shift) + (tok0 & (p.page_size - 1))));
    } else {
        const int past = p.seq_lens[c.b] - p.n_new;
        const int rows = p.rows_per_box;
        int npages = (past - tok0 + rows - 1) >> p.page_shift;
        const int max_pages = kTileTokens >> p.page_shift;
        npages = npages < max_pages ? npages : max_pages;
        mbar_arrive_expect_tx(bar, static_cast<uint32_t>(npages * rows * kRowBytes * 2));
        const int pg0 = tok0 >> p.page_shift;
        for (int r = 0; r < npages; ++r)
            four(r * rows, static_cast<int>(static_cast<long long>(page_at(p, row, pg0 + r)) << p.page_shift));
    }
}

template <int NWARPS, int NST>
__global__ void __launch_bounds__(NWARPS * 32, 1)
attn_partial_mma_kernel(const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
                        const AttnParams p) {
    extern __shared__ __align__(1024) uint8_t smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int r4 = lane >> 2, c4 = lane & 3;          // fragment row (and row + 8), column pair

    const int G = p.g_total / p.nsub;                 // query rows per record, <= 16
    const bool hi_rows = G > 8;
    const int nhs = p.nh_kv * p.nsub;
    int* s_cum = reinterpret_cast<int*>(smem + attn_dyn_smem_bytes<NWARPS, NST>() - kSelfScanBytes);
    const int* cum = tile_prefix(p, s_cum);
    const long long U = static_cast<long long>(cum[p.batch]) * nhs;
    const WarpSplit ws = warp_split(p, U);
    const long long qn = ws.qn;
    const int gw = logical_warp(ws, blockIdx.x, warp, NWARPS, gridDim.x);
    const long long u0 = static_cast<long long>(gw) * qn;
    const long long u1 = (u0 + qn < U) ? u0 + qn : U;
    if (u0 >= u1) return;
    const int depth = ring_depth<NWARPS, NST>(ws, U, blockIdx.x, gridDim.x);
    uint8_t* wbase = smem + static_cast<size_t>(warp) * depth * kStageBytes;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + static_cast<size_t>(NWARPS) * NST * kStageBytes) + warp * depth;

    if (lane == 0) {
        for (int s = 0; s < depth; ++s) mbar_init(&bars[s], 1);
        fence_mbar_init();
        fence_proxy_async_smem();
        tma_prefetch_desc(&tmK);
        tma_prefetch_desc(&tmV);
    }
    __syncwarp();

    TileCursor cc, pc;
    cc.cum = cum;
    cc.locate(p, u0, nhs);
    // Prologue: lane s starts the copies of stage s, so the page-table reads of all stages of the ring are one
    // round trip instead of a chain of them.
    if (lane < depth && u0 + lane < u1) {
        TileCursor c;
        c.cum = cum;
        c.locate(p, u0 + lane, nhs);
        issue_tile_sw(p, &tmK, &tmV, c, wbase + lane * kStageBytes, &bars[lane]);
    }
    long long pu = (u0 + depth < u1) ? u0 + depth : u1;  // next unit the producer (lane 0) will issue
    pc = cc;
    if (pu < u1) pc.locate(p, pu, nhs);
    __syncwarp();

    uint32_t phase_bits = 0;
    int stage = 0;
    bool failed = false;

    uint32_t qa[8][4];            // A fragments of the (zero-padded) 16 x 128 query block
    float o[16][4];               // O accumulators: 16 slices of 8 head-dim columns
    float m_lo = -INFINITY, m_hi = -INFINITY, l_lo = 0.f, l_hi = 0.f;
    int past_b = 0;
    bool seg_open = false;

    for (long long u = u0; u < u1; ++u) {
        if (!seg_open) {
            const int h = cc.hs / p.nsub, sub = cc.hs - h * p.nsub;
            const __nv_bfloat16* qrow =
                p.q + static_cast<long long>(cc.b) * p.q_stride + static_cast<long long>(h * p.g_total + sub * G) * kHeadDim;
            const bool v_lo = r4 < G, v_hi = r4 + 8 < G;
#pragma unroll
            for (int ks = 0; ks < 8; ++ks) {
                const int d0 = ks * 16 + 2 * c4;
                qa[ks][0] = v_lo ? *reinterpret_cast<const uint32_t*>(qrow + r4 * kHeadDim + d0) : 0u;
                qa[ks][2] = v_lo ? *reinterpret_cast<const uint32_t*>(qrow + r4 * kHeadDim + d0 + 8) : 0u;
                qa[ks][1] = v_hi ? *reinterpret_cast<const uint32_t*>(qrow + (r4 + 8) * kHeadDim + d0) : 0u;
                qa[ks][3] = v_hi ? *reinterpret_cast<const uint32_t*>(qrow + (r4 + 8) * kHeadDim + d0 + 8) : 0u;
            }
#pragma unroll
            for (int nt = 0; nt < 16; ++nt) o[nt][0] = o[nt][1] = o[nt][2] = o[nt][3] = 0.f;
            m_lo = m_hi = -INFINITY;
            l_lo = l_hi = 0.f;
            past_b = p.seq_lens[cc.b] - p.n_new;
            seg_open = true;
        }

        if (!__all_sync(0xffffffffu, mbar_wait_bounded(&bars[stage], (phase_bits >> stage) & 1u))) {
            failed = true;
            break;
        }
        phase_bits ^= (1u << stage);
        uint8_t* sK = wbase + stage * kStageBytes;
        uint8_t* sV = sK + 2 * kMmaHalfBytes;
        const uint32_t sK_a = smem_u32(sK), sV_a = smem_u32(sV);
        const int valid = past_b - cc.tile * kTileTokens;

        if (valid < kTileTokens) {
            // Rows past the request's last token may hold anything; their probabilities are zero, but the
            // tensor core still multiplies, so V must be finite there.
            for (int idx = lane; idx < (kTileTokens - valid) * 16; idx += 32)
                *reinterpret_cast<uint4*>(sV + sw_tile_off(valid + (idx >> 4), idx & 15)) = make_uint4(0, 0, 0, 0);
            fence_proxy_async_smem();   // these stores precede the next TMA write into the same stage
            __syncwarp();
        }

        // ---- S = Q K^T ----
        float s0[4] = {0.f, 0.f, 0.f, 0.f}, s1[4] = {0.f, 0.f, 0.f, 0.f};   // tokens 0-7, tokens 8-15
        {
            const int mi = lane >> 3, r = lane & 7;
            const int tok = (mi >> 1) * 8 + r;
#pragma unroll
            for (int ks = 0; ks < 8; ++ks) {
                uint32_t b[4];
                ldmatrix_x4(b, sK_a + sw_tile_off(tok, 2 * ks + (mi & 1)));
                mma_bf16_16816(s0, qa[ks], b[0], b[1]);
                mma_bf16_16816(s1, qa[ks], b[2], b[3]);
            }
        }
        // ---- online softmax: this lane holds tokens 2*c4, 2*c4+1 (s0) and 8+2*c4, 9+2*c4 (s1) of rows r4, r4+8 ----
        const bool t0 = 2 * c4 < valid, t1 = 2 * c4 + 1 < valid, t2 = 8 + 2 * c4 < valid, t3 = 9 + 2 * c4 < valid;
        float v_lo4[4] = {t0 ? s0[0] * p.scale_log2 : -INFINITY, t1 ? s0[1] * p.scale_log2 : -INFINITY,
                          t2 ? s1[0] * p.scale_log2 : -INFINITY, t3 ? s1[1] * p.scale_log2 : -INFINITY};
        float tm = fmaxf(fmaxf(v_lo4[0], v_lo4[1]), fmaxf(v_lo4[2], v_lo4[3]));
        tm = fmaxf(tm, __shfl_xor_sync(0xffffffffu, tm, 1));
        tm = fmaxf(tm, __shfl_xor_sync(0xffffffffu, tm, 2));
        const float mn_lo = fmaxf(m_lo, tm);
        const float mu_lo = (mn_lo == -INFINITY) ? 0.f : mn_lo;
        const float alpha_lo = exp2f(m_lo - mu_lo);
        const float p0 = exp2f(v_lo4[0] - mu_lo), p1 = exp2f(v_lo4[1] - mu_lo), p2 = exp2f(v_lo4[2] - mu_lo),
                    p3 = exp2f(v_lo4[3] - mu_lo);
        l_lo = l_lo * alpha_lo + (p0 + p1) + (p2 + p3);
        m_lo = mn_lo;
        uint32_t pa[4];
        pa[0] = pack_bf16x2(p0, p1);
        pa[2] = pack_bf16x2(p2, p3);
        pa[1] = 0u;
        pa[3] = 0u;
        float alpha_hi = 1.f;
        if (hi_rows) {
            float w4[4] = {t0 ? s0[2] * p.scale_log2 : -INFINITY, t1 ? s0[3] * p.scale_log2 : -INFINITY,
                           t2 ? s1[2] * p.scale_log2 : -INFINITY, t3 ? s1[3] * p.scale_log2 : -INFINITY};
            float th = fmaxf(fmaxf(w4[0], w4[1]), fmaxf(w4[2], w4[3]));
            th = fmaxf(th, __shfl_xor_sync(0xffffffffu, th, 1));
            th = fmaxf(th, __shfl_xor_sync(0xffffffffu, th, 2));
            const float mn_hi = fmaxf(m_hi, th);
            const float mu_hi = (mn_hi == -INFINITY) ? 0.f : mn_hi;
            alpha_hi = exp2f(m_hi - mu_hi);
            const float h0 = exp2f(w4[0] - mu_hi), h1 = exp2f(w4[1] - mu_hi), h2 = exp2f(w4[2] - mu_hi),
                        h3 = exp2f(w4[3] - mu_hi);
            l_hi = l_hi * alpha_hi + (h0 + h1) + (h2 + h3);
            m_hi = mn_hi;
            pa[1] = pack_bf16x2(h0, h1);
            pa[3] = pack_bf16x2(h2, h3);
        }
        // The running maximum rarely moves after the first tiles: skip the 64 multiplies when no row needs them.
        if (!__all_sync(0xffffffffu, alpha_lo == 1.f && alpha_hi == 1.f)) {
#pragma unroll
            for (int nt = 0; nt < 16; ++nt) {
                o[nt][0] *= alpha_lo;
                o[nt][1] *= alpha_lo;
                o[nt][2] *= alpha_hi;
                o[nt][3] *= alpha_hi;
            }
        }
        // ---- O += P V ----
        {
            const int mi = lane >> 3, r = lane & 7;
            const int tok = (mi & 1) * 8 + r;
#pragma unroll
            for (int n2 = 0; n2 < 8; ++n2) {
                uint32_t b[4];
                ldmatrix_x4_trans(b, sV_a + sw_tile_off(tok, 2 * n2 + (mi >> 1)));
                mma_bf16_16816(o[2 * n2], pa, b[0], b[1]);
                mma_bf16_16816(o[2 * n2 + 1], pa, b[2], b[3]);
            }
        }
        __syncwarp();

        if (pu < u1) {
            if (lane == 0) issue_tile_sw(p, &tmK, &tmV, pc, wbase + stage * kStageBytes, &bars[stage]);
            pc.advance(p, nhs);
            ++pu;
        }
        stage = (stage + 1 == depth) ? 0 : stage + 1;

        const bool last_of_seg = (cc.tile + 1 == cc.tiles_b) || (u + 1 == u1);
        if (last_of_seg) {
            const int seg = cc.b * nhs + cc.hs;
            float* out = p.partials + static_cast<size_t>(gw + seg) * (G * kPartialStride);
            float lt_lo = l_lo, lt_hi = l_hi;
            lt_lo += __shfl_xor_sync(0xffffffffu, lt_lo, 1);
            lt_lo += __shfl_xor_sync(0xffffffffu, lt_lo, 2);
            lt_hi += __shfl_xor_sync(0xffffffffu, lt_hi, 1);
            lt_hi += __shfl_xor_sync(0xffffffffu, lt_hi, 2);
            if (r4 < G) {
                float* og = out + r4 * kPartialStride;
#pragma unroll
                for (int nt = 0; nt < 16; ++nt)
                    *reinterpret_cast<float2*>(og + nt * 8 + 2 * c4) = make_float2(o[nt][0], o[nt][1]);
                if (c4 == 0) {
                    og[128] = m_lo;
                    og[129] = lt_lo;
                }
            }
            if (r4 + 8 < G) {
                float* og = out + (r4 + 8) * kPartialStride;
#pragma unroll
                for (int nt = 0; nt < 16; ++nt)
                    *reinterpret_cast<float2*>(og + nt * 8 + 2 * c4) = make_float2(o[nt][2], o[nt][3]);
                if (c4 == 0) {
                    og[128] = m_hi;
                    og[129] = lt_hi;
                }
            }
            seg_open = false;
        }
        cc.advance(p, nhs);
    }

    if (failed) {
        if (lane == 0) atomicOr(p.status, kStatusWaitTimeout | kStatusInStreaming);
        for (int s = 0; s < depth; ++s) (void)mbar_wait_bounded(&bars[s], (phase_bits >> s) & 1u);
    }
}

}  // namespace dkv

namespace dkv {

__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t a) {
    uint32_t d;
    asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(d) : "r"(a));
    return d;
}

// Variant for up to 8 query heads per KV head: the roles of the product are swapped, tokens (then head
// dimensions) on the 16-row M side and the query heads on the 8-column N side,
//
//   S^T[16 tokens x 8 q] = K_tile[16 x 128] . Q^T[128 x 8]        8 mma.m16n8k16 (A = K by ldmatrix, B = Q in registers)
//   O^T[128 d x 8 q]    += V_tile^T[128 x 16] . P^T[16 x 8]       8 mma.m16n8k16 (A = V by ldmatrix.trans, B = P^T)
//
// which halves the tensor-core instructions and the accumulator registers of the 16-row form above (O^T: 32
// registers, Q: 16), so that a 16-warp CTA stays near 100 registers per thread and leaves room on the SM for
// the decode projection.  P^T reaches its B-fragment layout with one movmatrix per 8 tokens.  The reference maximum
// of a query head is shared by the eight lanes that hold its columns; it moves only when some score exceeds it by
// more than 2^8 (one warp vote per tile), so the three-shuffle reduction runs on the first tiles only.
template <int NWARPS, int NST>
__global__ void __maxnreg__(NWARPS == 16 ? 104 : NWARPS == 12 ? 168 : 232)   // 16 warps: room for the decode projection
attn_partial_mma8_kernel(const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
                         const AttnParams p) {
    extern __shared__ __align__(1024) uint8_t smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int r4 = lane >> 2, c4 = lane & 3;

    const int G = p.g_total / p.nsub;                 // query heads per record, <= 8
    const int nhs = p.nh_kv * p.nsub;
    int* s_cum = reinterpret_cast<int*>(smem + attn_dyn_smem_bytes<NWARPS, NST>() - kSelfScanBytes);
    const int* cum = tile_prefix(p, s_cum);
    const long long U = static_cast<long long>(cum[p.batch]) * nhs;
    const WarpSplit ws = warp_split(p, U);
    const long long qn = ws.qn;
    const int gw = logical_warp(ws, blockIdx.x, warp, NWARPS, gridDim.x);
    const long long u0 = static_cast<long long>(gw) * qn;
    const long long u1 = (u0 + qn < U) ? u0 + qn : U;
    if (u0 >= u1) return;
    const int depth = ring_depth<NWARPS, NST>(ws, U, blockIdx.x, gridDim.x);
    uint8_t* wbase = smem + static_cast<size_t>(warp) * depth * kStageBytes;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + static_cast<size_t>(NWARPS) * NST * kStageBytes) + warp * depth;

    if (lane == 0) {
        for (int s = 0; s < depth; ++s) mbar_init(&bars[s], 1);
        fence_mbar_init();
        fence_proxy_async_smem();
        tma_prefetch_desc(&tmK);
        tma_prefetch_desc(&tmV);
    }
    __syncwarp();

    TileCursor cc, pc;
    cc.cum = cum;
    cc.locate(p, u0, nhs);
    // Prologue: lane s starts the copies of stage s, so the page-table reads of all stages of the ring are one
    // round trip instead of a chain of them.
    if (lane < depth && u0 + lane < u1) {
        TileCursor c;
        c.cum = cum;
        c.locate(p, u0 + lane, nhs);
        issue_tile_sw(p, &tmK, &tmV, c, wbase + lane * kStageBytes, &bars[lane]);
    }
    long long pu = (u0 + depth < u1) ? u0 + depth : u1;  // next unit the producer (lane 0) will issue
    pc = cc;
    if (pu < u1) pc.locate(p, pu, nhs);
    __syncwarp();

    uint32_t phase_bits = 0;
    int stage = 0;
    bool failed = false;

    uint32_t qb[8][2];            // B fragments of Q^T: query head r4, dims 16 ks + 2 c4 (+8)
    float o[8][4];                // O^T: dims 16 mt + r4 (+8) x query heads 2 c4, 2 c4 + 1
    float m0 = -INFINITY, m1 = -INFINITY;   // reference maxima of query heads 2 c4 and 2 c4 + 1 (same in all r4 lanes)
    float l0 = 0.f, l1 = 0.f;               // this lane's share of the sums (its tokens r4 and r4 + 8)
    int past_b = 0;
    bool seg_open = false;

    for (long long u = u0; u < u1; ++u) {
        if (!seg_open) {
            const int h = cc.hs / p.nsub, sub = cc.hs - h * p.nsub;
            const __nv_bfloat16* qrow =
                p.q + static_cast<long long>(cc.b) * p.q_stride + static_cast<long long>(h * p.g_total + sub * G + r4) * kHeadDim;
            const bool have = r4 < G;
#pragma unroll
            for (int ks = 0; ks < 8; ++ks) {
                qb[ks][0] = have ? *reinterpret_cast<const uint32_t*>(qrow + ks * 16 + 2 * c4) : 0u;
                qb[ks][1] = have ? *reinterpret_cast<const uint32_t*>(qrow + ks * 16 + 2 * c4 + 8) : 0u;
            }
#pragma unroll
            for (int mt = 0; mt < 8; ++mt) o[mt][0] = o[mt][1] = o[mt][2] = o[mt][3] = 0.f;
            m0 = m1 = -INFINITY;
            l0 = l1 = 0.f;
            past_b = p.seq_lens[cc.b] - p.n_new;
            seg_open = true;
        }

        if (!__all_sync(0xffffffffu, mbar_wait_bounded(&bars[stage], (phase_bits >> stage) & 1u))) {
            failed = true;
            break;
        }
        phase_bits ^= (1u << stage);
        uint8_t* sK = wbase + stage * kStageBytes;
        uint8_t* sV = sK + 2 * kMmaHalfBytes;
        const uint32_t sK_a = smem_u32(sK), sV_a = smem_u32(sV);
        const int valid = past_b - cc.tile * kTileTokens;

        if (valid < kTileTokens) {
            // Rows past the request's last token may hold anything; their probabilities are zero, but the
            // tensor core still multiplies, so V must be finite there.
            for (int idx = lane; idx < (kTileTokens - valid) * 16; idx += 32)
                *reinterpret_cast<uint4*>(sV + sw_tile_off(valid + (idx >> 4), idx & 15)) = make_uint4(0, 0, 0, 0);
            fence_proxy_async_smem();   // these stores precede the next TMA write into the same stage
            __syncwarp();
        }

        // ---- S^T = K Q^T: this lane gets tokens r4, r4 + 8 of query heads 2 c4, 2 c4 + 1 ----
        float s[4] = {0.f, 0.f, 0.f, 0.f};
        {
            const int mi = lane >> 3, r = lane & 7;
            const int tok = (mi & 1) * 8 + r;
#pragma unroll
            for (int ks = 0; ks < 8; ++ks) {
                uint32_t a[4];
                ldmatrix_x4(a, sK_a + sw_tile_off(tok, 2 * ks + (mi >> 1)));
                mma_bf16_16816(s, a, qb[ks][0], qb[ks][1]);
            }
        }
        const bool t_lo = r4 < valid, t_hi = r4 + 8 < valid;
        const float v00 = t_lo ? s[0] * p.scale_log2 : -INFINITY, v01 = t_lo ? s[1] * p.scale_log2 : -INFINITY;
        const float v10 = t_hi ? s[2] * p.scale_log2 : -INFINITY, v11 = t_hi ? s[3] * p.scale_log2 : -INFINITY;
        float x0 = fmaxf(v00, v10), x1 = fmaxf(v01, v11);
        const bool grow = (x0 > m0 + 8.f) || (x1 > m1 + 8.f) || (m0 == -INFINITY && x0 > -INFINITY) ||
                          (m1 == -INFINITY && x1 > -INFINITY);
        if (__any_sync(0xffffffffu, grow)) {
#pragma unroll
            for (int sh = 4; sh < 32; sh <<= 1) {
                x0 = fmaxf(x0, __shfl_xor_sync(0xffffffffu, x0, sh));
                x1 = fmaxf(x1, __shfl_xor_sync(0xffffffffu, x1, sh));
            }
            const float n0 = fmaxf(m0, x0), n1 = fmaxf(m1, x1);
            const float a0 = (n0 == -INFINITY) ? 1.f : exp2f(m0 - n0), a1 = (n1 == -INFINITY) ? 1.f : exp2f(m1 - n1);
            m0 = n0;
            m1 = n1;
            l0 *= a0;
            l1 *= a1;
#pragma unroll
            for (int mt = 0; mt < 8; ++mt) {
                o[mt][0] *= a0;
                o[mt][1] *= a1;
                o[mt][2] *= a0;
                o[mt][3] *= a1;
            }
        }
        const float u0m = (m0 == -INFINITY) ? 0.f : m0, u1m = (m1 == -INFINITY) ? 0.f : m1;
        const float p00 = exp2f(v00 - u0m), p01 = exp2f(v01 - u1m), p10 = exp2f(v10 - u0m), p11 = exp2f(v11 - u1m);
        l0 += p00 + p10;
        l1 += p01 + p11;
        // P^T (tokens x heads) in accumulator layout -> B fragments (token pairs of head r4) by transposing 8 x 8 blocks.
        const uint32_t pb0 = movmatrix_trans(pack_bf16x2(p00, p01));
        const uint32_t pb1 = movmatrix_trans(pack_bf16x2(p10, p11));
        // ---- O^T += V^T P^T ----
        {
            const int mi = lane >> 3, r = lane & 7;
            const int tok = (mi >> 1) * 8 + r;
#pragma unroll
            for (int mt = 0; mt < 8; ++mt) {
                uint32_t a[4];
                ldmatrix_x4_trans(a, sV_a + sw_tile_off(tok, 2 * mt + (mi & 1)));
                mma_bf16_16816(o[mt], a, pb0, pb1);
            }
        }
        __syncwarp();

        if (pu < u1) {
            if (lane == 0) issue_tile_sw(p, &tmK, &tmV, pc, wbase + stage * kStageBytes, &bars[stage]);
            pc.advance(p, nhs);
            ++pu;
        }
        stage = (stage + 1 == depth) ? 0 : stage + 1;

        const bool last_of_seg = (cc.tile + 1 == cc.tiles_b) || (u + 1 == u1);
        if (last_of_seg) {
            const int seg = cc.b * nhs + cc.hs;
            float* out = p.partials + static_cast<size_t>(gw + seg) * (G * kPartialStride);
            float lt0 = l0, lt1 = l1;
#pragma unroll
            for (int sh = 4; sh < 32; sh <<= 1) {
                lt0 += __shfl_xor_sync(0xffffffffu, lt0, sh);
                lt1 += __shfl_xor_sync(0xffffffffu, lt1, sh);
            }
            const int q0 = 2 * c4, q1 = 2 * c4 + 1;
            if (q0 < G) {
                float* og = out + q0 * kPartialStride;
#pragma unroll
                for (int mt = 0; mt < 8; ++mt) {
                    og[16 * mt + r4] = o[mt][0];
                    og[16 * mt + r4 + 8] = o[mt][2];
                }
                if (r4 == 0) {
                    og[128] = m0;
                    og[129] = lt0;
                }
            }
            if (q1 < G) {
                float* og = out + q1 * kPartialStride;
#pragma unroll
                for (int mt = 0; mt < 8; ++mt) {
                    og[16 * mt + r4] = o[mt][1];
                    og[16 * mt + r4 + 8] = o[mt][3];
                }
                if (r4 == 0) {
                    og[128] = m1;
                    og[129] = lt1;
                }
            }
            seg_open = false;
        }
        cc.advance(p, nhs);
    }

    if (failed) {
        if (lane == 0) atomicOr(p.status, kStatusWaitTimeout | kStatusInStreaming);
        for (int s = 0; s < depth; ++s) (void)mbar_wait_bounded(&bars[s], (phase_bits >> s) & 1u);
    }
}

}  // namespace dkv
