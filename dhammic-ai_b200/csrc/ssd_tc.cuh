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
    const float* tcum;
    const float* dtT;
    const float* D;
    const float* seed;   // init (modes 0,1) or dfinal (mode 2), (b,h,p,n) fp32, may be null
    float* out_state;    // final_state (modes 0,1) or dinit (mode 2), may be null
    CUtensorMap mY;   // y store (mode 0)
    CUtensorMap mS;   // state store: 2D [b*nt*h*128][64]
    int save_states;  // store the state entering every tile of the walk through mS
    float* gS;           // mode 2: (b,h,nt,8) per warp exp(S_k) <Q_k, H_k>
    float* rterm;        // mode 2: (2,b,h,T) halves of e_i * sum_p dY[i,p] (C_i . H_k[p,:])
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

}  // namespace tc
}  // namespace ssd
#include "ssd_tc_bwd.cuh"
