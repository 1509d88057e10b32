// Split-KV decode attention over a slot-indexed bf16 KV pool that lives either in
// host-pinned (mapped) memory or in HBM.
//
// Data layout: K and V pools are [n_slots, NH_kv, 128] bf16 (one 256-byte row per token and
// head), the layout of the reference's token pool (directkv/directkv_pool.py:96-130) and, with
// slot = row * row_stride + position, of its request pool (directkv/directkv_request_pool.py:66-76).
//
// Work decomposition: the past tokens of every (request, kv head) are cut into 16-token tiles;
// all tiles of the batch form one linear sequence that is divided evenly over all warps of the
// grid.  Each warp streams its tiles through a private ring of shared-memory stages filled by
// TMA (one 3-D box of 16 rows x 256 B per K or V tile, straight from the pool - over PCIe when
// the pool is host memory), keeps (m, l, O) of an online softmax in registers and writes one
// fp32 partial per (request, kv head) piece it touched.  A merge kernel combines the partials
// with the token decoded in this step (csrc/directKV_kernel.cuh:749-787 gives the algebra).
//
// Every wait is bounded; nothing traps.
#pragma once

#include "dkv_common.cuh"

namespace dkv {

constexpr int kHeadDim       = 128;
constexpr int kTileTokens    = 16;                              // tokens per streamed tile
constexpr int kRowBytes      = kHeadDim * 2;                    // one token, one head, bf16
constexpr int kTileBytes     = kTileTokens * kRowBytes;         // 4096: K or V of one tile
constexpr int kStageBytes    = 2 * kTileBytes;                  // K + V
constexpr int kPartialStride = 132;                             // 128 O + m + l + 2 pad (fp32)
constexpr int kMaxExchangeRanks = 8;                            // GPUs of one box

struct AttnParams {
    const __nv_bfloat16* q;        // query rows; row b starts at q + b * q_stride, then [NH_q, 128]
    long long q_stride;            // elements between consecutive (virtual) requests
    const int* page_table;         // [rows, pt_stride] page ids, or nullptr for contiguous rows
    const int* row_map;            // [B] page-table / pool row of request b, or nullptr (row = b)
    const int* seq_lens;           // [B] tokens attended by request b, INCLUDING n_new
    const int* cum_tiles;          // [B + 1] exclusive prefix sum of past tiles (written by prep)
    float* partials;               // [(total_warps + B * NH_kv * nsub), G, kPartialStride]
    unsigned int* status;
    int batch;
    int nh_q, nh_kv;
    int g_total;                   // NH_q / NH_kv
    int nsub;                      // g_total / G: q-head sub-groups that re-read the same KV
    int pt_stride;
    int pt_rows;                   // rows of the page table, or 0 when the caller did not say (row not checked)
    int page_size, page_shift;     // power of two (paged mode)
    int rows_per_box;              // min(16, page_size): rows one TMA box brings
    long long row_stride;          // contiguous mode: slots per pool row
    int n_new;                     // trailing tokens per request that are NOT read from the pool
    int total_warps;               // gridDim.x * warps per CTA of the partial kernel
    int min_units;                 // fewer (head-slot, tile) units per warp of the grid than this: a short step (warp_split)
    int self_scan;                 // 1: batch <= kSelfScanMax and no prep kernel ran - the kernels work out the tile
                                   // prefix sums from seq_lens themselves (cum_tiles is not read)
    float scale_log2;              // softmax scale * log2(e)
};

// Tile prefix sums of a small batch without the prep kernel: warp 0 of every CTA scans seq_lens into shared memory.
// On a short step the prep launch and the dependency on it are a fifth of the step.  Every thread of the CTA calls
// this before anything else that might return (it holds a CTA barrier).
constexpr int kSelfScanMax = 32;
constexpr int kSelfScanBytes = 256;                             // room for kSelfScanMax + 1 ints

// Dynamic shared memory of the streaming kernels: the stages, one mbarrier per stage, the CTA's own length scan.
// (No static shared memory there: the dynamic part is 1 KB-aligned, so a static array would cost a whole KB, and
// the 16-warp kernels share their SM with the decode projection to within a few hundred bytes.)
template <int NWARPS, int NST>
__host__ __device__ constexpr size_t attn_dyn_smem_bytes() {
    return static_cast<size_t>(NWARPS) * NST * kStageBytes + static_cast<size_t>(NWARPS) * NST * 8 + kSelfScanBytes;
}

__device__ __forceinline__ const int* tile_prefix(const AttnParams& p, int* s_cum) {
    if (!p.self_scan) return p.cum_tiles;
    if (threadIdx.x < 32) {
        const int b = threadIdx.x;
        int v = 0;
        if (b < p.batch) {
            const int past = p.seq_lens[b] - p.n_new;
            v = past > 0 ? (past + 15) / 16 : 0;
        }
        int x = v;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int y = __shfl_up_sync(0xffffffffu, x, o);
            if (b >= o) x += y;
        }
        s_cum[b + 1] = x;
        if (b == 0) s_cum[0] = 0;
    }
    __syncthreads();
    return s_cum;
}

// Units per warp of the streaming grid.  A short step (one 4K request: 2048 units for 2368 warps) would give every
// warp a single tile and the merge one record per tile; there the work goes to fewer warps, which are taken
// one per CTA in turn (spread) so that the rows still come through all SMs' load paths.
struct WarpSplit {
    long long qn;
    bool spread;
};
__device__ __forceinline__ WarpSplit warp_split(const AttnParams& p, long long U) {
    WarpSplit w;
    w.qn = (U + p.total_warps - 1) / p.total_warps;
    w.spread = w.qn < p.min_units;
    if (w.spread) {
        // A short step: fewer than min_units units per warp of the grid.  Measured over one to eight requests of 1K to
        // 32K tokens, the step is shortest with about eleven of a CTA's sixteen warps at work and at least two units
        // each (one 4K request of a Llama-3-8B layer: two units 13.2 us, five 14.3; 8192 units: four 30.7, five 29.1).
        const long long target = static_cast<long long>(p.total_warps) * 45 / 64;
        w.qn = (U + target - 1) / target;
        if (w.qn < 2) w.qn = 2;
    }
    return w;
}
// Ring depth of a warp.  Normally every warp owns NST stages.  On a short step (spread mode) only the first few
// warps of a CTA have work - warp w is active iff w * nctas + cta < (warps with work) - and the stages of the idle
// ones would lie unused while an active warp waits for one tile at a time: a whole memory round trip per 16
// tokens.  The active warps therefore share out all NWARPS * NST stages of the CTA (at most kMaxRingDepth each), so
// that a warp has its whole unit range in flight at once.  Active warp w uses stages [w * depth, (w + 1) * depth).
constexpr int kMaxRingDepth = 8;
template <int NWARPS, int NST>
__device__ __forceinline__ int ring_depth(const WarpSplit& w, long long U, int cta, int nctas) {
    if (!w.spread) return NST;
    const long long n_log = (U + w.qn - 1) / w.qn;                    // warps of the grid that have work
    long long n_act = (n_log - cta + nctas - 1) / nctas;              // ... of this CTA: warps 0 .. n_act - 1
    n_act = n_act < 1 ? 1 : (n_act > NWARPS ? NWARPS : n_act);
    int depth = (NWARPS * NST) / static_cast<int>(n_act);
    depth = depth > kMaxRingDepth ? kMaxRingDepth : depth;
    return depth < NST ? NST : depth;
}

// Logical index (position of the warp's unit range, and of its partial record) of a physical warp.
__device__ __forceinline__ int logical_warp(const WarpSplit& w, int cta, int warp, int nwarps, int nctas) {
    return w.spread ? warp * nctas + cta : cta * nwarps + warp;
}

// ---------------------------------------------------------------------------
// prep: tiles per request -> exclusive prefix sum; with n_new == 1 also the position and the
// destination slot of the token each request adds in this step.  One CTA.
// ---------------------------------------------------------------------------
struct PrepParams {
    const int* seq_lens;
    int batch;
    int n_new;
    int* cum_tiles;           // [batch + 1]
    // new-token bookkeeping (n_new == 1), any of these may be nullptr
    int* tok_pos;             // [batch] seq_len - 1
    int* tok_slot;            // [batch] slot the token is stored to, or -1
    const int* page_table;
    const int* row_map;
    const int* pos_offset;    // [batch] added to the RoPE position, or nullptr
    int pt_stride, pt_rows, page_size, page_shift;   // pt_rows: rows of the page table, 0 = not given
    long long row_stride;
    int save;
    unsigned int* status;     // receives kStatusBadPage when the new token's page lies outside the table
};

__global__ void __launch_bounds__(256) attn_prep_kernel(const PrepParams pp) {
    __shared__ int warp_tot[8];
    __shared__ int carry_s;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    if (tid == 0) carry_s = 0;
    __syncthreads();
    for (int base = 0; base < pp.batch; base += 256) {
        const int b = base + tid;
        int v = 0;
        if (b < pp.batch) {
            const int len = pp.seq_lens[b];
            const int past = len - pp.n_new;
            v = past > 0 ? (past + kTileTokens - 1) / kTileTokens : 0;
            if (pp.n_new && pp.tok_pos != nullptr) {
                const int pos = len - 1;
                long long slot = -1;
                if (pp.save && pos >= 0) {
                    const int row = pp.row_map ? pp.row_map[b] : b;
                    if (pp.page_table) {
                        const int pg = pos >> pp.page_shift;
                        if (pg >= pp.pt_stride || row < 0 || (pp.pt_rows > 0 && row >= pp.pt_rows)) {
                            if (pp.status != nullptr) atomicOr(pp.status, kStatusBadPage);   // the token is not stored
                        } else {
                            slot = (static_cast<long long>(pp.page_table[static_cast<long long>(row) * pp.pt_stride + pg])
                                    << pp.page_shift) + (pos & (pp.page_size - 1));
                        }
                    } else
                        slot = static_cast<long long>(row) * pp.row_stride + pos;
                }
                pp.tok_pos[b] = pos + (pp.pos_offset ? pp.pos_offset[b] : 0);
                pp.tok_slot[b] = static_cast<int>(slot);
            }
        }
        int x = v;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            int y = __shfl_up_sync(0xffffffffu, x, o);
            if (lane >= o) x += y;
        }
        if (lane == 31) warp_tot[warp] = x;
        __syncthreads();
        int woff = 0;
        for (int w = 0; w < warp; ++w) woff += warp_tot[w];
        const int carry = carry_s;
        if (b < pp.batch) pp.cum_tiles[b] = carry + woff + x - v;
        __syncthreads();
        if (tid == 255) carry_s = carry + woff + x;
        __syncthreads();
    }
    if (tid == 0) pp.cum_tiles[pp.batch] = carry_s;
}

// ---------------------------------------------------------------------------
// Cursor over the linear tile sequence: (request b, head-slot hs = h * nsub + sub, tile).
// ---------------------------------------------------------------------------
struct TileCursor {
    const int* cum;               // [B + 1] exclusive prefix sum of past tiles (global memory, or the CTA's own scan)
    int b, hs, tile, tiles_b;
    __device__ __forceinline__ void locate(const AttnParams& p, long long u, int nhs) {
        int lo = 0, hi = p.batch - 1;
        while (lo < hi) {
            const int mid = (lo + hi + 1) >> 1;
            if (static_cast<long long>(cum[mid]) * nhs <= u) lo = mid; else hi = mid - 1;
        }
        b = lo;
        tiles_b = cum[b + 1] - cum[b];
        const long long r = u - static_cast<long long>(cum[b]) * nhs;
        hs = tiles_b > 0 ? static_cast<int>(r / tiles_b) : 0;
        tile = tiles_b > 0 ? static_cast<int>(r % tiles_b) : 0;
    }
    __device__ __forceinline__ void advance(const AttnParams& p, int nhs) {
        if (++tile < tiles_b) return;
        tile = 0;
        if (++hs < nhs) return;
        hs = 0;
        do {
            ++b;
            tiles_b = b < p.batch ? cum[b + 1] - cum[b] : 1;
        } while (b < p.batch && tiles_b == 0);
    }
};

// Page-table entry (row, pg) with both indices held inside the table.  seq_lens and row_map are device data that
// no host code has seen: a length beyond pt_stride pages, or a row beyond the table, is reported in the status
// word and the nearest entry is read instead (wrong rows for that request, but no access outside the table).
__device__ __forceinline__ int page_at(const AttnParams& p, int row, int pg) {
    const bool bad = pg >= p.pt_stride || row < 0 || (p.pt_rows > 0 && row >= p.pt_rows);
    if (bad) {
        atomicOr(p.status, kStatusBadPage);
        pg = pg < p.pt_stride ? pg : p.pt_stride - 1;
        row = row < 0 ? 0 : (p.pt_rows > 0 && row >= p.pt_rows) ? p.pt_rows - 1 : row;
    }
    return p.page_table[static_cast<long long>(row) * p.pt_stride + pg];
}

// Lane 0 only: start the TMA copies of one tile into a stage.
__device__ __forceinline__ void issue_tile(const AttnParams& p, const CUtensorMap* tmK, const CUtensorMap* tmV,
                                           const TileCursor& c, uint8_t* stage, uint64_t* bar) {
    const int h = c.hs / p.nsub;
    const int tok0 = c.tile * kTileTokens;
    const int row = p.row_map ? p.row_map[c.b] : c.b;
    if (p.page_table == nullptr) {
        const long long slot0 = static_cast<long long>(row) * p.row_stride + tok0;
        mbar_arrive_expect_tx(bar, kStageBytes);
        tma_load_3d(stage, tmK, bar, 0, h, static_cast<int>(slot0));
        tma_load_3d(stage + kTileBytes, tmV, bar, 0, h, static_cast<int>(slot0));
    } else if (p.page_size >= kTileTokens) {
        const int page = page_at(p, row, tok0 >> p.page_shift);
        const long long slot0 = (static_cast<long long>(page) << p.page_shift) + (tok0 & (p.page_size - 1));
        mbar_arrive_expect_tx(bar, kStageBytes);
        tma_load_3d(stage, tmK, bar, 0, h, static_cast<int>(slot0));
        tma_load_3d(stage + kTileBytes, tmV, bar, 0, h, static_cast<int>(slot0));
    } else {
        const int past = p.seq_lens[c.b] - p.n_new;
        const int rows = p.rows_per_box;  // == page_size
        int npages = (past - tok0 + rows - 1) >> p.page_shift;
        const int max_pages = kTileTokens >> p.page_shift;
        npages = npages < max_pages ? npages : max_pages;
        mbar_arrive_expect_tx(bar, static_cast<uint32_t>(npages * rows * kRowBytes * 2));
        const int pg0 = tok0 >> p.page_shift;
        for (int r = 0; r < npages; ++r) {
            const long long slot0 = static_cast<long long>(page_at(p, row, pg0 + r)) << p.page_shift;
            tma_load_3d(stage + r * rows * kRowBytes, tmK, bar, 0, h, static_cast<int>(slot0));
            tma_load_3d(stage + kTileBytes + r * rows * kRowBytes, tmV, bar, 0, h, static_cast<int>(slot0));
        }
    }
}

// Pair-wise fp32 math.  With one or two query heads per KV head the packed two-wide FMA of sm_100 halves the
// FMA instruction count; with four, the register pairing it needs costs more than it saves (measured), so
// the components are computed separately there.
template <bool PACKED>
__device__ __forceinline__ float2 fma2(const float2 a, const float2 b, const float2 c) {
    if constexpr (PACKED) return __ffma2_rn(a, b, c);
    else return make_float2(fmaf(a.x, b.x, c.x), fmaf(a.y, b.y, c.y));
}
template <bool PACKED>
__device__ __forceinline__ float2 mul2(const float2 a, const float2 b) {
    if constexpr (PACKED) return __fmul2_rn(a, b);
    else return make_float2(a.x * b.x, a.y * b.y);
}

// ---------------------------------------------------------------------------
// Partial attention.  Lane (g4 = lane / 8, j = lane % 8) owns tokens t == g4 (mod 4) of each
// tile and the head-dim slices [8j, 8j+8) and [64+8j, 64+8j+8); a quarter-warp therefore reads
// 128 contiguous bytes of a row with each 16-byte shared load (no bank conflicts).
// ---------------------------------------------------------------------------
// The 16-warp instance shares its SM with the decode projection (128 threads x 96 registers): 512 x 104 + 128 x 96
// registers fill the file exactly, so it must stay at 104 (dkv_context_set "check_coresidency" verifies it).
template <int G, int NWARPS, int NST>
__global__ void __maxnreg__(NWARPS == 16 ? (G == 1 ? 104 : 128) : NWARPS == 12 ? 168 : 232)
attn_partial_kernel(const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
                    const AttnParams p) {
    extern __shared__ __align__(1024) uint8_t smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g4 = lane >> 3, j = lane & 7;

    int* s_cum = reinterpret_cast<int*>(smem + attn_dyn_smem_bytes<NWARPS, NST>() - kSelfScanBytes);
    const int* cum = tile_prefix(p, s_cum);
    const int nhs = p.nh_kv * p.nsub;
    const long long U = static_cast<long long>(cum[p.batch]) * nhs;
    const WarpSplit ws = warp_split(p, U);
    const long long qn = ws.qn;
    const int gw = logical_warp(ws, blockIdx.x, warp, NWARPS, gridDim.x);
    const long long u0 = static_cast<long long>(gw) * qn;
    const long long u1 = (u0 + qn < U) ? u0 + qn : U;
    if (u0 >= u1) return;  // warps are independent: no CTA-wide barrier follows
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
        issue_tile(p, &tmK, &tmV, c, wbase + lane * kStageBytes, &bars[lane]);
    }
    long long pu = (u0 + depth < u1) ? u0 + depth : u1;  // next unit the producer (lane 0) will issue
    pc = cc;
    if (pu < u1) pc.locate(p, pu, nhs);
    __syncwarp();

    uint32_t phase_bits = 0;  // bit s = parity to wait for on stage s
    int stage = 0;
    bool failed = false;

    // fp32 pairs: the math below uses the packed two-wide FMA of sm_100 (one instruction per pair).
    float2 qf[G][8];
    float2 O[G][8];
    float m[G], l[G];
    int past_b = 0;
    bool seg_open = false;

    for (long long u = u0; u < u1; ++u) {
        if (!seg_open) {
            // New (request, head-slot) piece: load and pre-scale its G query rows.
            const int h = cc.hs / p.nsub, sub = cc.hs - h * p.nsub;
            const __nv_bfloat16* qrow =
                p.q + static_cast<long long>(cc.b) * p.q_stride + static_cast<long long>(h * p.g_total + sub * G) * kHeadDim;
#pragma unroll
            for (int g = 0; g < G; ++g) {
                const uint4 a = *reinterpret_cast<const uint4*>(qrow + g * kHeadDim + 8 * j);
                const uint4 b2 = *reinterpret_cast<const uint4*>(qrow + g * kHeadDim + 64 + 8 * j);
                const uint32_t w[8] = {a.x, a.y, a.z, a.w, b2.x, b2.y, b2.z, b2.w};
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    qf[g][i] = make_float2(bf16lo(w[i]) * p.scale_log2, bf16hi(w[i]) * p.scale_log2);
                }
#pragma unroll
                for (int i = 0; i < 8; ++i) O[g][i] = make_float2(0.f, 0.f);
                m[g] = -INFINITY;
                l[g] = 0.f;
            }
            past_b = p.seq_lens[cc.b] - p.n_new;
            seg_open = true;
        }

        // ---- wait for this tile ----
        // The vote keeps the decision warp-uniform: the shuffles below need every lane.
        if (!__all_sync(0xffffffffu, mbar_wait_bounded(&bars[stage], (phase_bits >> stage) & 1u))) {
            failed = true;
            break;
        }
        phase_bits ^= (1u << stage);
        const uint8_t* sK = wbase + stage * kStageBytes;
        const uint8_t* sV = sK + kTileBytes;
        const int valid = past_b - cc.tile * kTileTokens;  // >= 1; may exceed 16

        // ---- S = q . k ----
        float s[G][4];
#pragma unroll
        for (int tt = 0; tt < 4; ++tt) {
            const int t = tt * 4 + g4;
            const uint4 ka = *reinterpret_cast<const uint4*>(sK + t * kRowBytes + 16 * j);
            const uint4 kb = *reinterpret_cast<const uint4*>(sK + t * kRowBytes + 128 + 16 * j);
            const uint32_t w[8] = {ka.x, ka.y, ka.z, ka.w, kb.x, kb.y, kb.z, kb.w};
            float2 kf[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) kf[i] = make_float2(bf16lo(w[i]), bf16hi(w[i]));
#pragma unroll
            for (int g = 0; g < G; ++g) {
                float2 a0 = make_float2(0.f, 0.f), a1 = make_float2(0.f, 0.f);
#pragma unroll
                for (int i = 0; i < 8; i += 2) {
                    a0 = fma2<(G <= 2)>(qf[g][i], kf[i], a0);
                    a1 = fma2<(G <= 2)>(qf[g][i + 1], kf[i + 1], a1);
                }
                float acc = (a0.x + a0.y) + (a1.x + a1.y);
                acc += __shfl_xor_sync(0xffffffffu, acc, 1);
                acc += __shfl_xor_sync(0xffffffffu, acc, 2);
                acc += __shfl_xor_sync(0xffffffffu, acc, 4);
                s[g][tt] = (t < valid) ? acc : -INFINITY;
            }
        }

        // ---- online softmax (base-2 domain) ----
        float pr[G][4];
#pragma unroll
        for (int g = 0; g < G; ++g) {
            float tm = fmaxf(fmaxf(s[g][0], s[g][1]), fmaxf(s[g][2], s[g][3]));
            tm = fmaxf(tm, __shfl_xor_sync(0xffffffffu, tm, 8));
            tm = fmaxf(tm, __shfl_xor_sync(0xffffffffu, tm, 16));
            const float m_new = fmaxf(m[g], tm);
            const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
            const float alpha = exp2f(m[g] - m_use);  // m = -inf -> 0
            float ps = 0.f;
#pragma unroll
            for (int tt = 0; tt < 4; ++tt) {
                pr[g][tt] = exp2f(s[g][tt] - m_use);
                ps += pr[g][tt];
            }
            l[g] = l[g] * alpha + ps;
            m[g] = m_new;
#pragma unroll
            for (int i = 0; i < 8; ++i) O[g][i] = mul2<(G <= 2)>(O[g][i], make_float2(alpha, alpha));
        }

        // ---- O += P . V ----
#pragma unroll
        for (int tt = 0; tt < 4; ++tt) {
            const int t = tt * 4 + g4;
            if (t < valid) {
                const uint4 va = *reinterpret_cast<const uint4*>(sV + t * kRowBytes + 16 * j);
                const uint4 vb = *reinterpret_cast<const uint4*>(sV + t * kRowBytes + 128 + 16 * j);
                const uint32_t w[8] = {va.x, va.y, va.z, va.w, vb.x, vb.y, vb.z, vb.w};
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const float2 v2 = make_float2(bf16lo(w[i]), bf16hi(w[i]));
#pragma unroll
                    for (int g = 0; g < G; ++g) O[g][i] = fma2<(G <= 2)>(make_float2(pr[g][tt], pr[g][tt]), v2, O[g][i]);
                }
            }
        }
        __syncwarp();  // every lane is done reading this stage

        // ---- refill the stage ----
        if (pu < u1) {
            if (lane == 0) issue_tile(p, &tmK, &tmV, pc, wbase + stage * kStageBytes, &bars[stage]);
            pc.advance(p, nhs);
            ++pu;
        }
        stage = (stage + 1 == depth) ? 0 : stage + 1;

        // ---- end of this (request, head-slot) piece? ----
        const bool last_of_seg = (cc.tile + 1 == cc.tiles_b) || (u + 1 == u1);
        if (last_of_seg) {
            const int seg = cc.b * nhs + cc.hs;
            float* out = p.partials + static_cast<size_t>(gw + seg) * (G * kPartialStride);
#pragma unroll
            for (int g = 0; g < G; ++g) {
                float lt = l[g];
                lt += __shfl_xor_sync(0xffffffffu, lt, 8);
                lt += __shfl_xor_sync(0xffffffffu, lt, 16);
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    float2 o = O[g][i];
                    o.x += __shfl_xor_sync(0xffffffffu, o.x, 8);
                    o.y += __shfl_xor_sync(0xffffffffu, o.y, 8);
                    o.x += __shfl_xor_sync(0xffffffffu, o.x, 16);
                    o.y += __shfl_xor_sync(0xffffffffu, o.y, 16);
                    O[g][i] = o;
                }
                if (g4 == 0) {
                    float* og = out + g * kPartialStride;
                    *reinterpret_cast<float4*>(og + 8 * j) = make_float4(O[g][0].x, O[g][0].y, O[g][1].x, O[g][1].y);
                    *reinterpret_cast<float4*>(og + 8 * j + 4) = make_float4(O[g][2].x, O[g][2].y, O[g][3].x, O[g][3].y);
                    *reinterpret_cast<float4*>(og + 64 + 8 * j) = make_float4(O[g][4].x, O[g][4].y, O[g][5].x, O[g][5].y);
                    *reinterpret_cast<float4*>(og + 64 + 8 * j + 4) =
                        make_float4(O[g][6].x, O[g][6].y, O[g][7].x, O[g][7].y);
                    if (j == 0) {
                        og[128] = m[g];
                        og[129] = lt;
                    }
                }
            }
            seg_open = false;
        }
        cc.advance(p, nhs);
    }

    if (failed) {
        if (lane == 0) atomicOr(p.status, kStatusWaitTimeout | kStatusInStreaming);
        // Give copies still in flight a bounded chance to land before the stages are released.
        for (int s = 0; s < depth; ++s) (void)mbar_wait_bounded(&bars[s], (phase_bits >> s) & 1u);
    }
}

// ---------------------------------------------------------------------------
// Merge: one warp per (request, q head); lane owns head-dim elements [4 lane, 4 lane + 4).
// Combines the partials of every warp that touched the (request, kv head) piece with the
// token decoded in this step (its K/V come from the projection kernel or from the caller).
// Output modes: normalised bf16 rows, and/or the unnormalised fp32 (O, m, l) triple used when
// the sequence is split across GPUs.
// ---------------------------------------------------------------------------
struct MergeParams {
    AttnParams a;
    int G;                           // q heads per partial record (template G of the partial kernel)
    const __nv_bfloat16* kv_new;     // [B, NH_kv, 2, 128] bf16 or nullptr (n_new == 0)
    __nv_bfloat16* out;              // [B, NH_q, 128] bf16 (row b at out + b * out_stride) or nullptr
    long long out_stride;
    float* lse;                      // [B, NH_q] natural-log LSE, or nullptr
    float* part_out;                 // [B, NH_q, kPartialStride] unnormalised partial, or nullptr
    // Sequence split without a collective call: the unnormalised record of every row is stored into the
    // exchange buffer of EVERY rank (plain stores over NVLink for peers) at [x_rank][row], then one
    // system-scope increment per row tells that rank how many rows of x_rank have landed.  The host passes
    // the half of each rank's double buffer (records and counters) that belongs to this step's parity, and the
    // step's sequence number, which travels in every record so that the consumer can tell a stale one.
    int x_world;                     // 0: off
    int x_rank;
    unsigned int x_tag;              // sequence number of the step (never 0)
    long long x_max_rows;
    float* x_part[kMaxExchangeRanks];            // rank p's buffer of this parity [x_world, x_max_rows, kPartialStride]
    unsigned int* x_count[kMaxExchangeRanks];    // rank p's arrival counters of this parity [x_world]
};

// WPR warps share one (request, query head) row: each takes blocks of 8 consecutive partial records (loads
// issued together, one running-maximum update per block) and warp 0 of the row folds the WPR results.  A long
// single request leaves hundreds of records per row (one per warp of the streaming grid), which a single warp
// reading them one after the other would turn into the longest kernel of the step.
constexpr int kMergeThreads = 256;
constexpr int kMergeBlock = 8;       // records loaded together

// WPR = 32 (a CTA of 1024 threads on one row) is for a single very long request: one record per warp of the
// streaming grid means about 300 per row at 128K tokens.
constexpr int merge_threads(int wpr) { return wpr > kMergeThreads / 32 ? wpr * 32 : kMergeThreads; }

template <int WPR>
__global__ void __launch_bounds__(merge_threads(WPR)) attn_merge_kernel(const MergeParams mp) {
    constexpr int kThreads = merge_threads(WPR);
    const AttnParams& p = mp.a;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int part = warp % WPR, row_in_cta = warp / WPR;
    __shared__ int s_cum[kSelfScanMax + 1];
    const int* cum = tile_prefix(p, s_cum);
    const long long wid = static_cast<long long>(blockIdx.x) * (kThreads / 32 / WPR) + row_in_cta;
    const bool row_valid = wid < static_cast<long long>(p.batch) * p.nh_q;
    if (WPR == 1 && !row_valid) return;
    const int b = row_valid ? static_cast<int>(wid / p.nh_q) : 0, hq = row_valid ? static_cast<int>(wid % p.nh_q) : 0;
    const int h = hq / p.g_total, gt = hq % p.g_total;
    const int sub = gt / mp.G, g = gt % mp.G;
    const int nhs = p.nh_kv * p.nsub;
    const int hs = h * p.nsub + sub;

    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    float m = -INFINITY, l = 0.f;

    // The row's query and the new token's K/V row depend on nothing that is read below: fetched first, they arrive
    // with the records instead of after them (one memory round trip less on a step that is a handful of them).
    const bool with_new = mp.kv_new != nullptr && p.n_new > 0 && (WPR == 1 || part == 0) && row_valid;
    const __nv_bfloat16* qrow = p.q + static_cast<long long>(b) * p.q_stride + static_cast<long long>(hq) * kHeadDim;
    uint2 qw = make_uint2(0u, 0u), kw = qw, vw = qw;
    if (with_new) {
        const __nv_bfloat16* kn = mp.kv_new + (static_cast<long long>(b) * p.nh_kv + h) * 2 * kHeadDim;
        qw = *reinterpret_cast<const uint2*>(qrow + 4 * lane);
        kw = *reinterpret_cast<const uint2*>(kn + 4 * lane);
        vw = *reinterpret_cast<const uint2*>(kn + kHeadDim + 4 * lane);
    }

    const int tiles_b = cum[b + 1] - cum[b];
    int n_parts = 1;              // warps of the row that found records to read
    if (row_valid && tiles_b > 0) {
        const long long U = static_cast<long long>(cum[p.batch]) * nhs;
        const long long qn = warp_split(p, U).qn;
        const long long s0 = static_cast<long long>(cum[b]) * nhs + static_cast<long long>(hs) * tiles_b;
        const long long e0 = s0 + tiles_b;
        const int seg = b * nhs + hs;
        const int gw_first = static_cast<int>(s0 / qn), gw_last = static_cast<int>((e0 - 1) / qn);
        const int n = gw_last - gw_first + 1;
        n_parts = (n + kMergeBlock - 1) / kMergeBlock;
        n_parts = n_parts > WPR ? WPR : n_parts;
        const float* rec0 = p.partials + static_cast<size_t>(gw_first + seg) * (mp.G * kPartialStride) + g * kPartialStride;
        const size_t rec_stride = static_cast<size_t>(mp.G) * kPartialStride;
        for (int base = part * kMergeBlock; base < n; base += WPR * kMergeBlock) {
            float mi[kMergeBlock], li[kMergeBlock];
            float4 oi[kMergeBlock];
#pragma unroll
            for (int j = 0; j < kMergeBlock; ++j) {
                const bool on = base + j < n;
                const float* rec = rec0 + static_cast<size_t>(on ? base + j : base) * rec_stride;
                const float2 ml = *reinterpret_cast<const float2*>(rec + 128);
                oi[j] = *reinterpret_cast<const float4*>(rec + 4 * lane);
                mi[j] = on ? ml.x : -INFINITY;
                li[j] = on ? ml.y : 0.f;
            }
            float mn = m;
#pragma unroll
            for (int j = 0; j < kMergeBlock; ++j) mn = fmaxf(mn, mi[j]);
            const float mu = (mn == -INFINITY) ? 0.f : mn;
            const float a = exp2f(m - mu);
            acc.x *= a;
            acc.y *= a;
            acc.z *= a;
            acc.w *= a;
            l *= a;
#pragma unroll
            for (int j = 0; j < kMergeBlock; ++j) {
                const float c = exp2f(mi[j] - mu);
                acc.x += oi[j].x * c;
                acc.y += oi[j].y * c;
                acc.z += oi[j].z * c;
                acc.w += oi[j].w * c;
                l += li[j] * c;
            }
            m = mn;
        }
    }

    if (WPR > 1) {
        __shared__ float4 s_acc[kThreads / 32][32];
        __shared__ float2 s_ml[kThreads / 32];
        s_acc[warp][lane] = acc;
        if (lane == 0) s_ml[warp] = make_float2(m, l);
        __syncthreads();
        if (part != 0 || !row_valid) return;
        // Fold only the warps that had records (a short step leaves a few dozen records for a row that 32 warps
        // were launched for); the order is fixed, so the result does not depend on WPR's choice.
        for (int j = 1; j < n_parts; ++j) {
            const float2 ml = s_ml[warp + j];
            const float4 oj = s_acc[warp + j][lane];
            const float mn = fmaxf(m, ml.x);
            const float mu = (mn == -INFINITY) ? 0.f : mn;
            const float a = exp2f(m - mu), c = exp2f(ml.x - mu);
            acc.x = acc.x * a + oj.x * c;
            acc.y = acc.y * a + oj.y * c;
            acc.z = acc.z * a + oj.z * c;
            acc.w = acc.w * a + oj.w * c;
            l = l * a + ml.y * c;
            m = mn;
        }
    }

    if (with_new) {
        float d = bf16lo(qw.x) * bf16lo(kw.x) + bf16hi(qw.x) * bf16hi(kw.x) + bf16lo(qw.y) * bf16lo(kw.y) +
                  bf16hi(qw.y) * bf16hi(kw.y);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) d += __shfl_xor_sync(0xffffffffu, d, o);
        const float sn = d * p.scale_log2;
        const float mn = fmaxf(m, sn);
        const float a = exp2f(m - mn), c = exp2f(sn - mn);
        acc.x = acc.x * a + bf16lo(vw.x) * c;
        acc.y = acc.y * a + bf16hi(vw.x) * c;
        acc.z = acc.z * a + bf16lo(vw.y) * c;
        acc.w = acc.w * a + bf16hi(vw.y) * c;
        l = l * a + c;
        m = mn;
    }

    if (mp.part_out != nullptr) {
        float* po = mp.part_out + (static_cast<long long>(b) * p.nh_q + hq) * kPartialStride;
        *reinterpret_cast<float4*>(po + 4 * lane) = acc;
        if (lane == 0) {
            po[128] = m;
            po[129] = l;
        }
    }
    if (mp.x_world > 0) {
        const long long row = static_cast<long long>(b) * p.nh_q + hq;
        for (int r = 0; r < mp.x_world; ++r) {
            float* po = mp.x_part[r] + (static_cast<long long>(mp.x_rank) * mp.x_max_rows + row) * kPartialStride;
            *reinterpret_cast<float4*>(po + 4 * lane) = acc;
            if (lane == 0) *reinterpret_cast<float4*>(po + 128) = make_float4(m, l, __uint_as_float(mp.x_tag), 0.f);
        }
        __threadfence_system();      // the record is visible system-wide before the count moves
        __syncwarp();
        if (lane < mp.x_world) atomicAdd_system(mp.x_count[lane] + mp.x_rank, 1u);
    }
    if (mp.out != nullptr) {
        const float inv = l > 0.f ? 1.f / l : 0.f;
        uint2 w;
        w.x = pack_bf16x2(acc.x * inv, acc.y * inv);
        w.y = pack_bf16x2(acc.z * inv, acc.w * inv);
        *reinterpret_cast<uint2*>(mp.out + static_cast<long long>(b) * mp.out_stride +
                                  static_cast<long long>(hq) * kHeadDim + 4 * lane) = w;
    }
    if (mp.lse != nullptr && lane == 0)
        mp.lse[static_cast<long long>(b) * p.nh_q + hq] = (l > 0.f) ? m * 0.6931471805599453f + logf(l) : -INFINITY;
}

// ---------------------------------------------------------------------------
// Merge of R unnormalised partial sets [R, rows, kPartialStride] (sequence split across GPUs,
// after the all-gather): one warp per row.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(128) merge_rank_partials_kernel(const float* __restrict__ parts, int nranks,
                                                                  long long rows, __nv_bfloat16* __restrict__ out,
                                                                  float* __restrict__ lse) {
    const int lane = threadIdx.x & 31;
    const long long r = static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (r >= rows) return;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    float m = -INFINITY, l = 0.f;
    for (int k = 0; k < nranks; ++k) {
        const float* rec = parts + (static_cast<long long>(k) * rows + r) * kPartialStride;
        const float mi = rec[128], li = rec[129];
        const float4 oi = *reinterpret_cast<const float4*>(rec + 4 * lane);
        const float mn = fmaxf(m, mi);
        const float mu = (mn == -INFINITY) ? 0.f : mn;
        const float a = exp2f(m - mu), c = exp2f(mi - mu);
        acc.x = acc.x * a + oi.x * c;
        acc.y = acc.y * a + oi.y * c;
        acc.z = acc.z * a + oi.z * c;
        acc.w = acc.w * a + oi.w * c;
        l = l * a + li * c;
        m = mn;
    }
    const float inv = l > 0.f ? 1.f / l : 0.f;
    uint2 w;
    w.x = pack_bf16x2(acc.x * inv, acc.y * inv);
    w.y = pack_bf16x2(acc.z * inv, acc.w * inv);
    *reinterpret_cast<uint2*>(out + r * kHeadDim + 4 * lane) = w;
    if (lse != nullptr && lane == 0) lse[r] = (l > 0.f) ? m * 0.6931471805599453f + logf(l) : -INFINITY;
}

// ---------------------------------------------------------------------------
// Consumer side of the exchange: one warp per row waits (bounded) until every rank's count says
// its records for this step have landed in THIS GPU's buffer, then merges them from local memory.
// ---------------------------------------------------------------------------
struct ExchangeMergeParams {
    const float* parts;                       // this rank's buffer of the step's parity [world, max_rows, kPartialStride]
    const unsigned int* count;                // this rank's arrival counters of that parity [world]
    unsigned int expected[kMaxExchangeRanks]; // cumulative rows each rank must have delivered on that parity
    unsigned int tag;                         // sequence number every record of this step carries
    int world;
    long long max_rows, rows;
    __nv_bfloat16* out;                       // [rows, 128]
    float* lse;                               // [rows] or nullptr
    unsigned int* status;
    unsigned long long wait_limit_ns;         // after this long without all records the kernel reports and returns
};

__device__ __forceinline__ unsigned int ld_acquire_sys(const unsigned int* p) {
    unsigned int v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

__global__ void __launch_bounds__(128) merge_exchange_kernel(const ExchangeMergeParams ep) {
    const int lane = threadIdx.x & 31;
    const long long r = static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (r >= ep.rows) return;
    // lane k watches rank k's counter
    bool ok = true;
    if (lane < ep.world) {
        // wrap-safe comparison: the counters only grow
        if (static_cast<int>(ld_acquire_sys(ep.count + lane) - ep.expected[lane]) < 0) {
            const unsigned long long t0 = globaltimer_ns();
            for (;;) {
                if (static_cast<int>(ld_acquire_sys(ep.count + lane) - ep.expected[lane]) >= 0) break;
                if (globaltimer_ns() - t0 > ep.wait_limit_ns) {
                    ok = false;
                    break;
                }
                __nanosleep(200);
            }
        }
    }
    ok = __all_sync(0xffffffffu, ok);
    if (!ok) {
        if (lane == 0) atomicOr(ep.status, kStatusWaitTimeout | kStatusInExchange);
        return;
    }
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    float m = -INFINITY, l = 0.f;
    bool stale = false;
    for (int k = 0; k < ep.world; ++k) {
        const float* rec = ep.parts + (static_cast<long long>(k) * ep.max_rows + r) * kPartialStride;
        const float4 ml = __ldcg(reinterpret_cast<const float4*>(rec + 128));
        const float4 oi = __ldcg(reinterpret_cast<const float4*>(rec + 4 * lane));
        stale |= (__float_as_uint(ml.z) != ep.tag);      // a record of another step: the ranks' calls do not line up
        const float mn = fmaxf(m, ml.x);
        const float mu = (mn == -INFINITY) ? 0.f : mn;
        const float a = exp2f(m - mu), c = exp2f(ml.x - mu);
        acc.x = acc.x * a + oi.x * c;
        acc.y = acc.y * a + oi.y * c;
        acc.z = acc.z * a + oi.z * c;
        acc.w = acc.w * a + oi.w * c;
        l = l * a + ml.y * c;
        m = mn;
    }
    if (stale && lane == 0) atomicOr(ep.status, kStatusExchangeOrder);
    const float inv = l > 0.f ? 1.f / l : 0.f;
    uint2 w;
    w.x = pack_bf16x2(acc.x * inv, acc.y * inv);
    w.y = pack_bf16x2(acc.z * inv, acc.w * inv);
    *reinterpret_cast<uint2*>(ep.out + r * kHeadDim + 4 * lane) = w;
    if (ep.lse != nullptr && lane == 0) ep.lse[r] = (l > 0.f) ? m * 0.6931471805599453f + logf(l) : -INFINITY;
}

}  // namespace dkv
