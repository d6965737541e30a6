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
//   walk_kernel<MODE>   one CTA per (batch, head) walks the tiles with the state (64 x 128 fp32)
//                       in registers:
//        MODE 0  forward:   Y = ((C B^T) o L) X + diag(e) C H^T (+ D x);  H <- e^{S} H + X^T diag(d) B
//        MODE 1  states:    only the recurrence; stores H_k (state entering tile k) as bf16
//        MODE 2  dstates:   reverse walk, Q <- e^{S} Q + dY^T diag(e) C; stores Q_k = dH_{k+1} as bf16
//   bwd_tile_kernel     one CTA per (batch, tile, group), heads of the group in an inner loop so
//                       that dB and dC accumulate over heads in TMEM:
//        dG = dY X^T, dS = dG o L, dX = G^T dY + diag(d) B Q^T, dC += dS B + diag(e) dY H,
//        dB += dS^T C + diag(d) X Q, and the per-position decay-gradient terms.
//
// TMEM lane = tile row; every epilogue is one thread per row (tcgen05.ld 32x32b).
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

inline bool supported(int dtype, int T, int h, int p, int n, int g, int l) {
    (void)h;
    (void)g;
    return dtype == 1 && p == HP && n == DN && T % LT == 0 && (l % LT == 0 || LT % l == 0);
}

// ------------------------------------------------------------------------------------------
__global__ void tile_cumsum_kernel(const float* __restrict__ cum, const float* __restrict__ dt, float* __restrict__ tcum,
                                   float* __restrict__ dtT, int b, int T, int h, int l) {
    const int t = blockIdx.x * blockDim.x + threadIdx.x;
    const int hh = blockIdx.y, bb = blockIdx.z;
    if (t >= T) return;
    const int c = T / l, k = t / l, i = t - k * l;
    const float* cu = cum + ((size_t)((size_t)bb * h + hh) * c) * l;
    float v = cu[(size_t)k * l + i];
    if (l >= LT) {
        const int i0 = (i / LT) * LT;
        if (i0 > 0) v -= cu[(size_t)k * l + i0 - 1];
    } else {
        const int k0 = (t / LT) * (LT / l);
        for (int kk = k0; kk < k; ++kk) v += cu[(size_t)kk * l + l - 1];
    }
    const size_t o = ((size_t)bb * h + hh) * T + t;
    tcum[o] = v * 1.4426950408889634f;  // stored in log2 units: every consumer uses exp2
    if (dt) dtT[o] = dt[((size_t)bb * T + t) * h + hh];
}

// ------------------------------------------------------------------------------------------
struct WalkParams {
    CUtensorMap mU;   // x (modes 0,1) or dy (mode 2): 2D [b*T][h*64]
    CUtensorMap mV;   // B (modes 0,1) or C (mode 2):  2D [b*T][g*128]
    CUtensorMap mC;   // C (mode 0)
    CUtensorMap mY;   // y store (mode 0)
    CUtensorMap mS;   // state store (modes 1,2): 2D [b*nt*h*128][64]
    const float* tcum;
    const float* dtT;
    const float* D;
    const float* seed;   // init (modes 0,1) or dfinal (mode 2), (b,h,p,n) fp32, may be null
    float* out_state;    // final_state (modes 0,1) or dinit (mode 2), may be null
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
namespace ssd {
namespace tc {

// ------------------------------------------------------------------------------------------
struct BwdParams {
    CUtensorMap mX, mdY, mB, mC;   // loads: [b*T][h*64] and [b*T][g*128]
    CUtensorMap mH, mQ;            // loads: states [b*nt*h*128][64]
    CUtensorMap mdX, mdB, mdC;     // stores
    const float* tcum;
    const float* dtT;
    const float* D;
    float* g;        // (b,h,T)  g_row - g_col
    float* ddtx;     // (b,h,T)  sum_p dX_eff * x
    float* dyx;      // (b,h,T)  sum_p dy * x
    int* status;
    int T, h, hpg, nt;
};

__global__ void __launch_bounds__(128, 1) bwd_tile_kernel(const __grid_constant__ BwdParams P) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* sm = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* sC = sm;                  // 2 panels [pos][n]
    uint8_t* sB = sC + 2 * PANEL;      // 2 panels [pos][n]
    uint8_t* sX = sB + 2 * PANEL;      // [pos][p]
    uint8_t* sdY = sX + PANEL;         // [pos][p]
    uint8_t* sH = sdY + PANEL;         // [n][p]  state entering the tile
    uint8_t* sQ = sH + PANEL;          // [n][p]  gradient of the state leaving the tile
    uint8_t* sG = sQ + PANEL;          // 2 panels [i][j]   (C B^T) o L ; later staging
    uint8_t* sdS = sG + 2 * PANEL;     // 2 panels [i][j]   dG o L o dt ; later staging
    float* scum = reinterpret_cast<float*>(sdS + 2 * PANEL);
    float* sdt = scum + LT;
    __shared__ uint64_t bar_cb, bar_ld, bar_m1, bar_m2;
    __shared__ uint32_t tmem_slot;
    __shared__ int failed;
    __shared__ float sred[4];

    const int tid = threadIdx.x, warp = tid >> 5;
    const int k = blockIdx.x, gg = blockIdx.y, bb = blockIdx.z;
    const int row0 = bb * P.T + k * LT;

    if (tid == 0) {
        failed = 0;
        mbar_init(&bar_cb, 1);
        mbar_init(&bar_ld, 1);
        mbar_init(&bar_m1, 1);
        mbar_init(&bar_m2, 1);
        mbar_fence_init();
    }
    if (warp == 0) {
        tmem_alloc(&tmem_slot, 512);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tm = tmem_slot;
    // phase 1: S [0,128) dG [128,256); phase 2 (aliases): dX1 [0,64) dX2 [64,128) Yoff [128,192)
    // dYe (bf16 pairs) [192,224) Xd (bf16 pairs) [224,256); persistent over heads: dC [256,384) dB [384,512)
    const uint32_t tS = tm, tdG = tm + 128, tX1 = tm, tX2 = tm + 64, tYo = tm + 128, tdYe = tm + 192, tXd = tm + 224,
                   tdC = tm + 256, tdB = tm + 384;
    const uint32_t lanes = lane_base(warp);

    auto issue_head_loads = [&](int hh) {
        const int srow = (int)((((size_t)bb * P.nt + k) * P.h + hh) * DN);
        mbar_expect_tx(&bar_ld, 4 * PANEL);
        tma_load_2d(sX, &P.mX, &bar_ld, hh * HP, row0);
        tma_load_2d(sdY, &P.mdY, &bar_ld, hh * HP, row0);
        tma_load_2d(sH, &P.mH, &bar_ld, 0, srow);
        tma_load_2d(sQ, &P.mQ, &bar_ld, 0, srow);
    };
    if (tid == 0) {
        mbar_expect_tx(&bar_cb, 4 * PANEL);
        tma_load_2d(sC, &P.mC, &bar_cb, gg * DN, row0);
        tma_load_2d(sC + PANEL, &P.mC, &bar_cb, gg * DN + 64, row0);
        tma_load_2d(sB, &P.mB, &bar_cb, gg * DN, row0);
        tma_load_2d(sB + PANEL, &P.mB, &bar_cb, gg * DN + 64, row0);
        issue_head_loads(gg * P.hpg);
    }
    mbar_wait(&bar_cb, 0, &failed);

    for (int hl = 0; hl < P.hpg; ++hl) {
        const int hh = gg * P.hpg + hl;
        const uint32_t ph = hl & 1;
        const size_t bh = (size_t)bb * P.h + hh;
        const size_t tpos = bh * P.T + (size_t)k * LT + tid;
        const float cumv = P.tcum[tpos];
        const float dtv = P.dtT ? P.dtT[tpos] : 1.f;
        __syncthreads();  // previous head finished with scum / sdt and the staging buffers
        scum[tid] = cumv;
        sdt[tid] = dtv;
        if (tid == 0) tma_store_wait_read();
        mbar_wait(&bar_ld, ph, &failed);
        __syncthreads();
        const float Sk = scum[LT - 1];
        const uint32_t c0 = smem_u32(sC), b0 = smem_u32(sB), x0 = smem_u32(sX), y0 = smem_u32(sdY), h0 = smem_u32(sH),
                       q0 = smem_u32(sQ), g0 = smem_u32(sG), s0 = smem_u32(sdS);
        if (tid == 0) {
            tc_fence_after();
#pragma unroll
            for (int kk = 0; kk < 8; ++kk) {  // S = C B^T, K = n
                const uint32_t off = (kk >> 2) * PANEL + (kk & 3) * 32;
                mma_ss(tS, smem_desc(c0 + off, 16, 1024), smem_desc(b0 + off, 16, 1024), kIdescKK128, kk > 0);
            }
#pragma unroll
            for (int kk = 0; kk < 4; ++kk)  // dG = dY X^T, K = p
                mma_ss(tdG, smem_desc(y0 + kk * 32, 16, 1024), smem_desc(x0 + kk * 32, 16, 1024), kIdescKK128, kk > 0);
            mma_commit(&bar_m1);
        }
        // rows of x and dy of this thread (raw), kept for the epilogue
        uint32_t xr[32], yr[32];
#pragma unroll
        for (int ch = 0; ch < 8; ++ch) {
            uint4 v = *reinterpret_cast<const uint4*>(sX + sw128(tid, ch));
            xr[ch * 4 + 0] = v.x; xr[ch * 4 + 1] = v.y; xr[ch * 4 + 2] = v.z; xr[ch * 4 + 3] = v.w;
            uint4 u = *reinterpret_cast<const uint4*>(sdY + sw128(tid, ch));
            yr[ch * 4 + 0] = u.x; yr[ch * 4 + 1] = u.y; yr[ch * 4 + 2] = u.z; yr[ch * 4 + 3] = u.w;
        }
        const float ei = exp2f(cumv);
        const float dj = exp2f(Sk - cumv);
        float dyx = 0.f;
#pragma unroll
        for (int q = 0; q < 32; ++q) {
            float2 fx = __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&xr[q]));
            float2 fy = __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&yr[q]));
            dyx += fx.x * fy.x + fx.y * fy.y;
        }
        // <Q_k, H_k> over this thread's state row (n = tid): the gradient of the inter-tile decay exp(S_k)
        float qh = 0.f;
#pragma unroll
        for (int ch = 0; ch < 8; ++ch) {
            uint4 hv = *reinterpret_cast<const uint4*>(sH + sw128(tid, ch));
            uint4 qv = *reinterpret_cast<const uint4*>(sQ + sw128(tid, ch));
            const uint32_t* hu = reinterpret_cast<const uint32_t*>(&hv);
            const uint32_t* qu = reinterpret_cast<const uint32_t*>(&qv);
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                float2 fh = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&hu[q]));
                float2 fq = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&qu[q]));
                qh += fh.x * fq.x + fh.y * fq.y;
            }
        }
        mbar_wait(&bar_m1, ph, &failed);
        tc_fence_after();
        float rowacc = 0.f;
#pragma unroll 1
        for (int cb = 0; cb < LT; cb += 32) {
            float gv[32], dv[32];
            if (cb <= warp * 32) {
                uint32_t rs[32], rg[32];
                tmem_ld32(tS + lanes + cb, rs);
                tmem_ld32(tdG + lanes + cb, rg);
                tmem_ld_wait();
#pragma unroll
                for (int q = 0; q < 32; ++q) {
                    const int j = cb + q;
                    const float Lv = (j <= tid) ? exp2f(cumv - scum[j]) : 0.f;
                    const float dg = __uint_as_float(rg[q]) * sdt[j];
                    gv[q] = __uint_as_float(rs[q]) * Lv;
                    dv[q] = dg * Lv;
                    // the same bf16-rounded G that the dX product uses, so that row and column sums
                    // of dG o G cancel exactly
                    rowacc += dg * __bfloat162float(__float2bfloat16_rn(gv[q]));
                }
            } else {
#pragma unroll
                for (int q = 0; q < 32; ++q) { gv[q] = 0.f; dv[q] = 0.f; }
            }
            store_row32(sG + (cb >> 6) * PANEL, tid, cb & 63, gv);
            store_row32(sdS + (cb >> 6) * PANEL, tid, cb & 63, dv);
        }
        // A operands held in TMEM: dYe = e_i * dY and Xd = d_j * dt_j * x, bf16 pairs, 32 columns each
        {
            uint32_t a[32], bq[32];
            const float wx = dj * dtv;
#pragma unroll
            for (int q = 0; q < 32; ++q) {
                float2 fy = __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&yr[q]));
                float2 fx = __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&xr[q]));
                a[q] = pack_bf16(fy.x * ei, fy.y * ei);
                bq[q] = pack_bf16(fx.x * wx, fx.y * wx);
            }
            tmem_st32(tdYe + lanes, a);
            tmem_st32(tXd + lanes, bq);
            tmem_st_wait();
        }
        tc_fence_before();
        fence_async_smem();
        __syncthreads();
        if (tid == 0) {
            tc_fence_after();
#pragma unroll
            for (int kk = 0; kk < 8; ++kk)  // dX1 = G^T dY : A = G as MN-major (M = j), B = dY MN-major, K = i
                mma_ss(tX1, smem_desc(g0 + kk * 2048, PANEL, 1024), smem_desc(y0 + kk * 2048, PANEL, 1024), kIdescMM,
                       kk > 0);
#pragma unroll
            for (int kk = 0; kk < 8; ++kk) {  // dX2 = B Q^T : A = B K-major (K = n), B = Q^T [n][p] MN-major
                const uint32_t off = (kk >> 2) * PANEL + (kk & 3) * 32;
                mma_ss(tX2, smem_desc(b0 + off, 16, 1024), smem_desc(q0 + kk * 2048, PANEL, 1024), kIdescKM, kk > 0);
            }
#pragma unroll
            for (int kk = 0; kk < 8; ++kk) {  // Yoff = C H^T
                const uint32_t off = (kk >> 2) * PANEL + (kk & 3) * 32;
                mma_ss(tYo, smem_desc(c0 + off, 16, 1024), smem_desc(h0 + kk * 2048, PANEL, 1024), kIdescKM, kk > 0);
            }
#pragma unroll
            for (int kk = 0; kk < 8; ++kk) {  // dC += dS B : A = dS K-major (K = j), B = B [j][n] MN-major, N = 128
                const uint32_t off = (kk >> 2) * PANEL + (kk & 3) * 32;
                mma_ss(tdC, smem_desc(s0 + off, 16, 1024), smem_desc(b0 + kk * 2048, PANEL, 1024), kIdescKM128,
                       hl > 0 || kk > 0);
            }
#pragma unroll
            for (int kk = 0; kk < 4; ++kk)  // dC += dYe H : A = dYe in TMEM (K = p), B = H^T [n][p] K-major, N = 128
                mma_ts(tdC, tdYe + kk * 8, smem_desc(h0 + kk * 32, 16, 1024), kIdescKK128, true);
#pragma unroll
            for (int kk = 0; kk < 8; ++kk)  // dB += dS^T C : A = dS MN-major (M = j, K = i), B = C [i][n] MN-major
                mma_ss(tdB, smem_desc(s0 + kk * 2048, PANEL, 1024), smem_desc(c0 + kk * 2048, PANEL, 1024), kIdescMM128,
                       hl > 0 || kk > 0);
#pragma unroll
            for (int kk = 0; kk < 4; ++kk)  // dB += Xd Q : A = Xd in TMEM (K = p), B = Q^T [n][p] K-major
                mma_ts(tdB, tXd + kk * 8, smem_desc(q0 + kk * 32, 16, 1024), kIdescKK128, true);
            mma_commit(&bar_m2);
        }
        mbar_wait(&bar_m2, ph, &failed);
        tc_fence_after();
        if (tid == 0 && hl + 1 < P.hpg) issue_head_loads(hh + 1);
        // per-row epilogue: dx, ddtx, g
        {
            const float Dh = P.D ? P.D[hh] : 0.f;
            float ddt_acc = 0.f, yo_acc = 0.f, st_acc = 0.f;
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                uint32_t a[32], b2[32], o[32];
                tmem_ld32(tX1 + lanes + half * 32, a);
                tmem_ld32(tX2 + lanes + half * 32, b2);
                tmem_ld32(tYo + lanes + half * 32, o);
                tmem_ld_wait();
                float dxv[32];
#pragma unroll
                for (int q = 0; q < 16; ++q) {
                    float2 fx = __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&xr[half * 16 + q]));
                    float2 fy = __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&yr[half * 16 + q]));
                    const float e0 = __uint_as_float(a[2 * q]) + dj * __uint_as_float(b2[2 * q]);
                    const float e1 = __uint_as_float(a[2 * q + 1]) + dj * __uint_as_float(b2[2 * q + 1]);
                    ddt_acc += e0 * fx.x + e1 * fx.y;
                    st_acc += __uint_as_float(b2[2 * q]) * fx.x + __uint_as_float(b2[2 * q + 1]) * fx.y;
                    yo_acc += __uint_as_float(o[2 * q]) * fy.x + __uint_as_float(o[2 * q + 1]) * fy.y;
                    dxv[2 * q] = e0 * dtv + Dh * fy.x;
                    dxv[2 * q + 1] = e1 * dtv + Dh * fy.y;
                }
                store_row32(sG, tid, half * 32, dxv);
            }
            // gradient with respect to the tile-cumulative log-decay at this position; the terms that
            // act through S_k = cum[127] (state weights d_j and the inter-tile decay) go to the last row
            const float gi = rowacc + ei * yo_acc - dtv * ddt_acc;
            float red = dj * dtv * st_acc + exp2f(Sk) * qh;
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) red += __shfl_xor_sync(0xffffffffu, red, o);
            if ((tid & 31) == 0) sred[warp] = red;
            if (tid != LT - 1) P.g[tpos] = gi;
            P.ddtx[tpos] = ddt_acc;
            P.dyx[tpos] = dyx;
            tc_fence_before();
            fence_async_smem();
            __syncthreads();
            if (tid == LT - 1) P.g[tpos] = gi + sred[0] + sred[1] + sred[2] + sred[3];
        }
        if (tid == 0) {
            tma_store_2d(&P.mdX, sG, hh * HP, row0);
            tma_store_commit();
        }
    }
    // group outputs: dC and dB rows -> bf16 -> staging (sG, sdS) -> TMA store
    if (tid == 0) tma_store_wait_read();
    __syncthreads();
#pragma unroll 1
    for (int cb = 0; cb < DN; cb += 32) {
        uint32_t a[32], b2[32];
        tmem_ld32(tdC + lanes + cb, a);
        tmem_ld32(tdB + lanes + cb, b2);
        tmem_ld_wait();
        float va[32], vb[32];
#pragma unroll
        for (int q = 0; q < 32; ++q) { va[q] = __uint_as_float(a[q]); vb[q] = __uint_as_float(b2[q]); }
        store_row32(sG + (cb >> 6) * PANEL, tid, cb & 63, va);
        store_row32(sdS + (cb >> 6) * PANEL, tid, cb & 63, vb);
    }
    tc_fence_before();
    fence_async_smem();
    __syncthreads();
    if (tid == 0) {
        tma_store_2d(&P.mdC, sG, gg * DN, row0);
        tma_store_2d(&P.mdC, sG + PANEL, gg * DN + 64, row0);
        tma_store_2d(&P.mdB, sdS, gg * DN, row0);
        tma_store_2d(&P.mdB, sdS + PANEL, gg * DN + 64, row0);
        tma_store_commit();
        tma_store_wait_all();
        if (failed) atomicExch(P.status, 1);
    }
    __syncthreads();
    if (warp == 0) tmem_dealloc(tm, 512);
}

constexpr size_t kBwdSmem = 12 * PANEL + 2 * LT * 4 + 1024;

}  // namespace tc
}  // namespace ssd
