// Tensor-core path of the SSD chunked scan for sm_100a: tcgen05.mma with TMEM accumulators,
// operands staged in 128-byte-swizzled shared memory by TMA (no cluster multicast).
//
// Covered shapes: bf16 storage, headdim 64, d_state 128, sequence a multiple of 128, chunk a
// multiple or a divisor of 128.  The kernels work on tiles of 128 positions whatever the chunk
// size (the recurrence does not depend on where chunk boundaries fall); `tcum` is the inclusive
// cumulative log-decay inside each 128-tile.
//
// Kernels
//   tile_cumsum_kernel  a_cumsum (b,h,c,l) -> tcum (b,h,T), dt (b,T,h) -> dtT (b,h,T)
//   cumsum_tile_fused_kernel  the same together with the cumulative sums themselves, for chunk = 128
//   fwd_walk_kernel     one CTA per (batch, head) walks the tiles with the state (64 x 128 fp32) in registers:
//                       Y = ((C B^T) o L) X + diag(e) C H^T (+ D x);  H <- e^{S} H + X^T diag(d) B
//   states_walk_kernel  only the recurrence; stores H_k (state entering tile k) as bf16
//   summary_kernel      what a whole piece of the sequence adds to the state after it / to the state gradient
//                       before it (the quantities the sequence-parallel schedule exchanges): a stream, no recurrence
//   rev_walk_kernel     reverse walk of the backward pass, Q <- e^{S} Q + dY^T diag(e) C, software-pipelined
//                       over tiles; reads dY and C only, stores Q_k = dH_{k+1} as bf16
//   bwd_tile_kernel     persistent over (batch, tile, group) items, heads of the group in an inner loop so
//                       that dB and dC accumulate over heads in TMEM:
//        dG = dY X^T, dS = dG o L, dX = G^T dY + diag(d) B Q^T, dC += dS B + diag(e) dY H,
//        dB += dS^T C + diag(d) X Q, and the per-position decay-gradient terms.
//
// TMEM lane = tile row; every epilogue is one thread per row (tcgen05.ld 32x32b).  In the walk and the tile kernels one
// lane of a warp of its own issues the products and one lane of another warp the TMA copies.
#pragma once
#include "ssd_common.cuh"
#include "ssd_ptx.cuh"
#include "ssd_simt.cuh"

namespace ssd {
namespace tc {

using namespace ssd::ptx;

constexpr int LT = 128;  // tile length
constexpr int HP = 64;   // headdim
constexpr int DN = 128;  // d_state
constexpr int PANEL = 16384;  // bytes of one [128 rows][64 bf16] swizzled panel
// The decay mask of a 32-column block is the product of a per-row and a per-column factor taken relative to the
// block's last column.  Below the diagonal both are <= 1.  Inside the diagonal block the row factor is
// 2^(decay from the row to the block end) >= 1 and the column factor its inverse scale; beyond this many log2
// units across a block one of them would leave the fp32 range.  tile_cumsum_kernel raises a flag when any block
// of the call exceeds it, and the kernels that build the mask carry two bodies: the factorised one, and one that
// evaluates diagonal blocks entry by entry (one exp2 per entry); the flag selects the body on the device.
constexpr float kMaskSafeLog2 = 100.f;

inline bool supported(int dtype, int T, int h, int p, int n, int g, int l) {
    (void)h;
    (void)g;
    return dtype == 1 && p == HP && n == DN && T % LT == 0 && (l % LT == 0 || LT % l == 0);
}

// ------------------------------------------------------------------------------------------
// Tile-cumulative log2 decay and dt in (b,h,T) order, one block per (128-tile, 32 heads, batch): dt arrives in the
// caller's (b,T,h) order and goes through a shared-memory transpose, so reads and writes are both 128-byte rows.
__global__ void __launch_bounds__(256) tile_cumsum_kernel(const float* __restrict__ cum, const float* __restrict__ dt,
                                                          float* __restrict__ tcum, float* __restrict__ dtT,
                                                          const float* __restrict__ skip, float* __restrict__ skipT,
                                                          int* __restrict__ extreme, int b, int T, int h, int l) {
    __shared__ float sdt[LT][33];
    __shared__ float ssk[LT][33];
    const int kt = blockIdx.x, hg = blockIdx.y, bb = blockIdx.z;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int h0 = hg * 32;
    (void)b;
    if (dt) {
        const bool head_ok = h0 + lane < h;
#pragma unroll
        for (int t = warp; t < LT; t += 8)
            sdt[t][lane] = head_ok ? dt[((size_t)bb * T + (size_t)kt * LT + t) * h + h0 + lane] : 0.f;
    }
    if (skip) {  // per-position skip coefficient of the scaled operator form, same transpose
        const bool head_ok = h0 + lane < h;
#pragma unroll
        for (int t = warp; t < LT; t += 8)
            ssk[t][lane] = head_ok ? skip[((size_t)bb * T + (size_t)kt * LT + t) * h + h0 + lane] : 0.f;
    }
    __syncthreads();
    const int c = T / l;
#pragma unroll
    for (int i4 = 0; i4 < 4; ++i4) {
        const int hl = warp * 4 + i4, hh = h0 + hl;
        if (hh >= h) break;  // warp-uniform
        const float* cu = cum + ((size_t)((size_t)bb * h + hh) * c) * l;
        const size_t o = ((size_t)bb * h + hh) * T + (size_t)kt * LT;
#pragma unroll
        for (int s4 = 0; s4 < 4; ++s4) {
            const int tt = s4 * 32 + lane, t = kt * LT + tt;
            const int k = t / l, i = t - k * l;
            float v = cu[(size_t)k * l + i];
            if (l >= LT) {
                const int i0 = (i / LT) * LT;
                if (i0 > 0) v -= cu[(size_t)k * l + i0 - 1];
            } else {
                const int k0 = kt * (LT / l);
                for (int kk = k0; kk < k; ++kk) v += cu[(size_t)kk * l + l - 1];
            }
            v *= 1.4426950408889634f;  // stored in log2 units: every consumer uses exp2
            tcum[o + tt] = v;
            // decay across this 32-position block (lane 0 to lane 31)
            const float span = __shfl_sync(0xffffffffu, v, 0) - __shfl_sync(0xffffffffu, v, 31);
            if (lane == 0 && !(span <= kMaskSafeLog2)) atomicOr(extreme, 1);
            if (dt) dtT[o + tt] = sdt[tt][hl];
            if (skip) skipT[o + tt] = ssk[tt][hl];
        }
    }
}

// ------------------------------------------------------------------------------------------
// The two kernels above in one, for chunk size = tile size (128): reads the per-position log-decay once (dt * A_head,
// or `a` as given, fp32 or bf16) in the caller's (b,T,h) layout through a shared-memory transpose, scans it inside each
// 128-tile (warp per head, four 32-lane segments) and writes a_cumsum (b,h,c,l) in natural-log units, the same in
// log2 units (tcum), dt and skip in (b,h,T) order, and the extreme-decay flag.
// CH positions per pass: 128 (one pass) when there is no skip array to transpose, 64 (two passes, the running sums
// carried over) with it — three [CH][33] arrays must fit the 48 KB of static shared memory.
template <int CH, bool SKIP>
__global__ void __launch_bounds__(256) cumsum_tile_fused_kernel(const void* __restrict__ a, int a_is_bf16,
                                                                const float* __restrict__ dt, const float* __restrict__ A_head,
                                                                float* __restrict__ cum, float* __restrict__ tcum,
                                                                float* __restrict__ dtT, const float* __restrict__ skip,
                                                                float* __restrict__ skipT, int* __restrict__ extreme, int T, int h) {
    __shared__ float sa[CH][33];
    __shared__ float sdt[CH][33];
    __shared__ float ssk[SKIP ? CH : 1][33];
    const int kt = blockIdx.x, hg = blockIdx.y, bb = blockIdx.z;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int h0 = hg * 32;
    const bool head_ok = h0 + lane < h;
    const float Ah = (!a && head_ok) ? A_head[h0 + lane] : 0.f;
    float carry[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int part = 0; part < LT / CH; ++part) {
        if (part) __syncthreads();
#pragma unroll
        for (int t = warp; t < CH; t += 8) {
            const size_t i = ((size_t)bb * T + (size_t)kt * LT + part * CH + t) * h + h0 + lane;
            float d = 0.f, av = 0.f;
            if (head_ok) {
                if (dt) d = dt[i];
                if (a) av = a_is_bf16 ? __bfloat162float(((const __nv_bfloat16*)a)[i]) : ((const float*)a)[i];
                else av = d * Ah;
                if (SKIP) ssk[t][lane] = skip[i];
            }
            sa[t][lane] = av;
            sdt[t][lane] = d;
        }
        __syncthreads();
#pragma unroll
        for (int i4 = 0; i4 < 4; ++i4) {
            const int hl = warp * 4 + i4, hh = h0 + hl;
            if (hh >= h) break;  // warp-uniform
            const size_t o = ((size_t)bb * h + hh) * T + (size_t)kt * LT + part * CH;  // (b,h,T) = (b,h,c,l), l = 128
#pragma unroll
            for (int s2 = 0; s2 < CH / 32; ++s2) {
                const int tt = s2 * 32 + lane;
                float incl = sa[tt][hl];
#pragma unroll
                for (int of = 1; of < 32; of <<= 1) {
                    const float u = __shfl_up_sync(0xffffffffu, incl, of);
                    if (lane >= of) incl += u;
                }
                incl += carry[i4];
                carry[i4] = __shfl_sync(0xffffffffu, incl, 31);
                cum[o + tt] = incl;
                const float v = incl * 1.4426950408889634f;
                tcum[o + tt] = v;
                const float span = __shfl_sync(0xffffffffu, v, 0) - __shfl_sync(0xffffffffu, v, 31);
                if (lane == 0 && !(span <= kMaskSafeLog2)) atomicOr(extreme, 1);
                if (dt) dtT[o + tt] = sdt[tt][hl];
                if (SKIP) skipT[o + tt] = ssk[tt][hl];
            }
        }
    }
}

// ------------------------------------------------------------------------------------------
// Decay gradient of the tensor-core backward, one block per (128-tile, 32 heads, batch).
// Inputs in (b,h,T) layout (coalesced along t): the per-row gradients g w.r.t. the tile-cumulative
// log-decay, ddtx = sum_p dX x, dyx = sum_p dy x, and gS, the terms that act through the tile's last row.  Within a tile
//   dA[t] = sum_{t' >= t} g[t']      (a suffix sum, four 32-lane segments per warp and head)
// and  ddt = ddtx + dA A_head,  dA_head += dA dt,  dD += dyx.  dt is read and ddt / da written in the
// caller's (b,T,h) layout through a shared-memory transpose, so both sides are 128-byte rows.
struct DecayTileParams {
    const float* g;      // (b,h,T)
    const float* ddtx;   // (b,h,T)
    const float* dyx;    // (b,h,T) or null
    const float* gS;     // (b,h,nt,8) from the backward tile kernel: terms that act through the tile's last row
    const float* dt;     // (b,T,h) or null (operator form)
    const float* A_head; // (h) or null; null with dt given = scaled operator form (outputs ddt = ddtx, da, dskip = dyx)
    float* ddt;          // (b,T,h) or null
    float* da;           // (b,T,h) or null
    float* dskip;        // (b,T,h) or null (scaled operator form)
    float* dAh_part;     // (b*nt, h)
    float* dD_part;      // (b*nt, h) or null
    int b, T, h, nt;
};

__global__ void __launch_bounds__(256) decay_tile_kernel(DecayTileParams P) {
    __shared__ float sdt[LT][33];
    __shared__ float sout[LT][33];
    const int k = blockIdx.x, hg = blockIdx.y, bb = blockIdx.z;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int h0 = hg * 32;
    const bool head_ok = h0 + lane < P.h;
    if (P.dt) {
#pragma unroll
        for (int t = warp; t < LT; t += 8)
            sdt[t][lane] = head_ok ? P.dt[((size_t)bb * P.T + (size_t)k * LT + t) * P.h + h0 + lane] : 0.f;
    }
    // every load of the warp's four heads is issued before any of them is used
    const bool scaled = P.dt && !P.A_head;  // scaled operator form: three per-position outputs
    float va[4][4], dxa[4][4], yxp[4][4], gsa[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int hh = h0 + warp * 4 + i;
        gsa[i] = 0.f;
#pragma unroll
        for (int s4 = 0; s4 < 4; ++s4) va[i][s4] = dxa[i][s4] = yxp[i][s4] = 0.f;
        if (hh < P.h) {
            const size_t base = ((size_t)bb * P.h + hh) * P.T + (size_t)k * LT;
#pragma unroll
            for (int s4 = 0; s4 < 4; ++s4) {
                const int t = s4 * 32 + lane;
                va[i][s4] = P.g[base + t];
                dxa[i][s4] = P.ddtx[base + t];
                if (P.dyx) yxp[i][s4] = P.dyx[base + t];
            }
            if (lane < 8)  // the eight terms that act through the tile's last row, one per lane
                gsa[i] = P.gS[((((size_t)bb * P.h + hh) * P.nt) + k) * 8 + lane];
        }
    }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int hl = warp * 4 + i, hh = h0 + hl;
        if (hh >= P.h) break;  // warp-uniform
        float v[4];
#pragma unroll
        for (int s4 = 0; s4 < 4; ++s4) v[s4] = va[i][s4];
        {
            float gs = gsa[i];  // fixed-order sum of the eight terms (the other lanes hold zero), result in every lane
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) gs += __shfl_xor_sync(0xffffffffu, gs, o);
            if (lane == 31) v[3] += gs;
        }
        // suffix sums: inside each 32-lane segment by shuffles, then the totals of the later segments
        float tot[4];
#pragma unroll
        for (int s4 = 0; s4 < 4; ++s4) {
            float incl = v[s4];
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const float u = __shfl_down_sync(0xffffffffu, incl, o);
                if (lane + o < 32) incl += u;
            }
            v[s4] = incl;
            tot[s4] = __shfl_sync(0xffffffffu, incl, 0);
        }
        v[2] += tot[3];
        v[1] += tot[3] + tot[2];
        v[0] += (tot[3] + tot[2]) + tot[1];
#pragma unroll
        for (int s4 = 0; s4 < 4; ++s4) va[i][s4] = v[s4];  // d a[t] of this head and tile
        if (P.dt && !scaled) {
            float dAh = 0.f, yx = 0.f;
#pragma unroll
            for (int s4 = 0; s4 < 4; ++s4) {
                dAh += v[s4] * sdt[s4 * 32 + lane][hl];
                yx += yxp[i][s4];
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                dAh += __shfl_xor_sync(0xffffffffu, dAh, o);
                yx += __shfl_xor_sync(0xffffffffu, yx, o);
            }
            if (lane == 0) {
                const size_t po = ((size_t)bb * P.nt + k) * P.h + hh;
                P.dAh_part[po] = dAh;
                if (P.dD_part) P.dD_part[po] = yx;
            }
        }
    }
    // per-position outputs in the caller's (b,T,h) layout, one transpose through shared memory each:
    //   Mamba-2 form: ddt = ddtx + da A_head;  operator form: da;  scaled operator form: ddt = ddtx, da, dskip = dyx
    for (int pass = 0; pass < 3; ++pass) {
        float* out = nullptr;
        if (pass == 0) out = P.dt ? P.ddt : P.da;
        else if (pass == 1) out = scaled ? P.da : nullptr;
        else out = scaled ? P.dskip : nullptr;
        if (!out) continue;  // block-uniform
        __syncthreads();
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int hl = warp * 4 + i, hh = h0 + hl;
            if (hh >= P.h) break;
            const float Ah = (P.A_head && pass == 0) ? P.A_head[hh] : 0.f;
#pragma unroll
            for (int s4 = 0; s4 < 4; ++s4) {
                float val;
                if (pass == 0) val = P.dt ? dxa[i][s4] + va[i][s4] * Ah : va[i][s4];
                else if (pass == 1) val = va[i][s4];
                else val = yxp[i][s4];
                sout[s4 * 32 + lane][hl] = val;
            }
        }
        __syncthreads();
        if (head_ok) {
#pragma unroll
            for (int t = warp; t < LT; t += 8) out[((size_t)bb * P.T + (size_t)k * LT + t) * P.h + h0 + lane] = sout[t][lane];
        }
    }
}

// out[hh] = sum_r part[r, hh] over `rows` rows, one block per head, fixed summation tree (deterministic).
// A second (part, out) pair, when given, is reduced by the blocks with blockIdx.y = 1 of the same launch.
__global__ void __launch_bounds__(256) reduce_rows_kernel(const float* __restrict__ part, float* __restrict__ out, int rows, int h,
                                                          const float* __restrict__ part2 = nullptr, float* __restrict__ out2 = nullptr) {
    __shared__ float red[8];
    const int hh = blockIdx.x;
    if (blockIdx.y) {
        part = part2;
        out = out2;
    }
    float s = 0.f;
    for (int r = threadIdx.x; r < rows; r += 256) s += part[(size_t)r * h + hh];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = s;
    __syncthreads();
    if (threadIdx.x == 0) out[hh] = ((red[0] + red[1]) + (red[2] + red[3])) + ((red[4] + red[5]) + (red[6] + red[7]));
}

// ------------------------------------------------------------------------------------------
// Self-test of the bounded wait: one warp waits (a few thousand polls) on an mbarrier that nothing ever arrives at,
// gives up, records it in the status word exactly as the tile kernels do, and returns.  The context stays usable.
__global__ void __launch_bounds__(32) bounded_wait_selftest_kernel(int* status, int polls) {
    __shared__ uint64_t bar;
    __shared__ int failed;
    if (threadIdx.x == 0) {
        failed = 0;
        mbar_init(&bar, 1);
        mbar_fence_init();
    }
    __syncwarp();
    mbar_wait(&bar, 0, &failed, (uint32_t)polls);
    __syncwarp();
    if (threadIdx.x == 0 && failed) atomicExch(status, 1);
}

// ------------------------------------------------------------------------------------------
struct WalkParams {
    CUtensorMap mU;   // x (modes 0,1) or dy (reverse walks): 2D [b*T][h*64]
    CUtensorMap mV;   // B (modes 0,1) or C (reverse walks):  2D [b*T][g*128]
    CUtensorMap mC;   // C (mode 0)
    const float* tcum;
    const float* dtT;
    const float* D;
    const float* skipT;  // (b,h,T) per-position skip coefficient (replaces D), or null
    const float* seed;   // init (modes 0,1) or dfinal (reverse walks), (b,h,p,n) fp32, may be null
    float* out_state;    // final_state (modes 0,1) or dinit (reverse walks), may be null
    CUtensorMap mY;   // y store (mode 0)
    CUtensorMap mS;   // state store: 2D [b*nt*h*128][64]
    int save_states;  // store the state entering every tile of the walk through mS
    const int* extreme;  // see kMaskSafeLog2 (forward only)
    float* ysq;          // (b, T/128, h, 2, 128) per half row sum_p y^2 (forward only), or null
    int* status;
    int T, h, hpg, nt;
};

constexpr uint32_t kIdescS = instr_desc(128, 128, false, false);    // K-major x K-major, N = 128
constexpr uint32_t kIdescKM = instr_desc(128, 64, false, true);     // A K-major, B MN-major, N = 64
constexpr uint32_t kIdescMM = instr_desc(128, 64, true, true);      // both MN-major, N = 64
constexpr uint32_t kIdescKK128 = instr_desc(128, 128, false, false);
constexpr uint32_t kIdescKM128 = instr_desc(128, 128, false, true);  // A K-major, B MN-major, N = 128
constexpr uint32_t kIdescMM128 = instr_desc(128, 128, true, true);   // both MN-major, N = 128
constexpr uint32_t kIdescKK64 = instr_desc(128, 64, false, false);

__device__ __forceinline__ uint32_t lane_base(int warp) { return ((uint32_t)((warp & 3) * 32)) << 16; }

// Scale one 128-byte row of bf16 (8 chunks of 16 bytes) by w while copying src -> dst (both swizzled).
__device__ __forceinline__ void scale_row(const uint8_t* src, uint8_t* dst, int row, float w) {
#pragma unroll
    for (int ch = 0; ch < 8; ++ch) {
        uint4 v = *reinterpret_cast<const uint4*>(src + sw128(row, ch));
        uint32_t* u = reinterpret_cast<uint32_t*>(&v);
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            __nv_bfloat162 bv = *reinterpret_cast<__nv_bfloat162*>(&u[q]);
            float2 f = __bfloat1622float2(bv);
            u[q] = pack_bf16(f.x * w, f.y * w);
        }
        *reinterpret_cast<uint4*>(dst + sw128(row, ch)) = v;
    }
}

// Write 32 fp32 values (columns c0 .. c0+31 of this thread's row) as bf16 into a swizzled panel.
__device__ __forceinline__ void store_row32(uint8_t* panel, int row, int col0_in_panel, const float (&v)[32]) {
#pragma unroll
    for (int ch = 0; ch < 4; ++ch) {
        uint4 o;
        o.x = pack_bf16(v[ch * 8 + 0], v[ch * 8 + 1]);
        o.y = pack_bf16(v[ch * 8 + 2], v[ch * 8 + 3]);
        o.z = pack_bf16(v[ch * 8 + 4], v[ch * 8 + 5]);
        o.w = pack_bf16(v[ch * 8 + 6], v[ch * 8 + 7]);
        *reinterpret_cast<uint4*>(panel + sw128(row, col0_in_panel / 8 + ch)) = o;
    }
}

}  // namespace tc
}  // namespace ssd
#include "ssd_tc_walk.cuh"
#include "ssd_tc_fwd.cuh"
#include "ssd_tc_revwalk.cuh"
#include "ssd_tc_summary.cuh"
#include "ssd_tc_bwd.cuh"
