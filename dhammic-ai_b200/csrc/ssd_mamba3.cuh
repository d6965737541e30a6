// Element-wise prologue of the Mamba-3 style variant: data-dependent rotary state angles and the
// trapezoidal two-term products, forward and backward.  These are the steps the reference's block
// runs before its two scan calls (src/mamba_base_engine.py:128-181; rotation as in
// tests/kernels/test_rope.py:31-43; gamma / beta as in src/kernels/trapezoidal.py:6-12):
//
//   cum      = -cumsum_T(raw_angles)                                   (b,T,h,n/2)   scan_T kernels
//   Br, Cr   = rope(B_group(h), cum), rope(C_group(h), cum)            (b,T,h,n)     rope_fwd_kernel
//   Bprev[t] = Br[t-1]  (zero at t = 0)
//   dA = dt A_head,  gamma = lam dt,  beta = (1-lam) dt exp(dA)        (b,T,h)
//   xg = x gamma,  xb[t] = x[t-1] beta[t]                              (b,T,h,p)     xprod_fwd_kernel
//
// All of them are HBM-bound streaming kernels; the scans along T are two-pass (per-segment sums, then a
// segment-local scan seeded by the prefix of the earlier segments).
#pragma once
#include "ssd_common.cuh"

namespace ssd {
namespace m3 {

constexpr int SEG = 128;  // positions per scan segment

// ------------------------------------------------------------------------------------------
// Scan along T of a (b, T, E) tensor.  Pass 1: per-segment sums.
// ------------------------------------------------------------------------------------------
template <class T>
__global__ void __launch_bounds__(256) scanT_segsum_kernel(const T* __restrict__ in, float* __restrict__ segsum, int Tlen,
                                                           int E) {
    const int seg = blockIdx.x, bb = blockIdx.z;
    const int e = blockIdx.y * 256 + threadIdx.x;
    if (e >= E) return;
    const int nseg = gridDim.x;
    const int t0 = seg * SEG, t1 = min(Tlen, t0 + SEG);
    const T* p = in + ((size_t)bb * Tlen + t0) * E + e;
    float s = 0.f;
    for (int t = t0; t < t1; ++t, p += E) s += to_f(*p);
    segsum[((size_t)bb * nseg + seg) * E + e] = s;
}

// Pass 2: out[t] = sign * (sum over the segments before (after, if reverse) + running sum inside the segment).
template <class TI, class TO>
__global__ void __launch_bounds__(256) scanT_apply_kernel(const TI* __restrict__ in, const float* __restrict__ segsum,
                                                          TO* __restrict__ out, int Tlen, int E, int reverse, float sign) {
    const int seg = blockIdx.x, bb = blockIdx.z;
    const int e = blockIdx.y * 256 + threadIdx.x;
    if (e >= E) return;
    const int nseg = gridDim.x;
    float run = 0.f;
    if (!reverse) {
        for (int s = 0; s < seg; ++s) run += segsum[((size_t)bb * nseg + s) * E + e];
    } else {
        for (int s = nseg - 1; s > seg; --s) run += segsum[((size_t)bb * nseg + s) * E + e];
    }
    const int t0 = seg * SEG, t1 = min(Tlen, t0 + SEG);
    if (!reverse) {
        for (int t = t0; t < t1; ++t) {
            const size_t o = ((size_t)bb * Tlen + t) * E + e;
            run += to_f(in[o]);
            out[o] = from_f<TO>(sign * run);
        }
    } else {
        for (int t = t1 - 1; t >= t0; --t) {
            const size_t o = ((size_t)bb * Tlen + t) * E + e;
            run += to_f(in[o]);
            out[o] = from_f<TO>(sign * run);
        }
    }
}

// ------------------------------------------------------------------------------------------
// Rotation.  One block per (position, batch); thread e <-> (head, pair index m).
// ------------------------------------------------------------------------------------------
__device__ __forceinline__ void sincos_reduced(float a, float* s, float* c) {
    // reduce to [-pi, pi] first: the fast sine / cosine are accurate there
    const float k = rintf(a * 0.15915494309189535f);
    const float r = fmaf(-k, 6.283185307179586f, a);
    __sincosf(r, s, c);
}

template <class T>
__global__ void __launch_bounds__(256) rope_fwd_kernel(const T* __restrict__ B, const T* __restrict__ C,
                                                       const float* __restrict__ cum, T* __restrict__ Br,
                                                       T* __restrict__ Cr, T* __restrict__ Bprev, int Tlen, int h, int g,
                                                       int n) {
    const int t = blockIdx.x, bb = blockIdx.y;
    const int half = n / 2, hpg = h / g;
    const size_t row = (size_t)bb * Tlen + t;
    for (int e = threadIdx.x; e < h * half; e += 256) {
        const int hh = e / half, m = e - hh * half;
        const int gg = hh / hpg;
        float s, c;
        sincos_reduced(cum[row * h * half + e], &s, &c);
        const size_t ib = (row * g + gg) * n + m;
        const float b1 = to_f(B[ib]), b2 = to_f(B[ib + half]);
        const float c1 = to_f(C[ib]), c2 = to_f(C[ib + half]);
        const size_t o = (row * h + hh) * n + m;
        const T br1 = from_f<T>(b1 * c - b2 * s), br2 = from_f<T>(b1 * s + b2 * c);
        Br[o] = br1;
        Br[o + half] = br2;
        Cr[o] = from_f<T>(c1 * c - c2 * s);
        Cr[o + half] = from_f<T>(c1 * s + c2 * c);
        if (t + 1 < Tlen) {
            Bprev[o + (size_t)h * n] = br1;
            Bprev[o + (size_t)h * n + half] = br2;
        }
        if (t == 0) {
            Bprev[o] = from_f<T>(0.f);
            Bprev[o + half] = from_f<T>(0.f);
        }
    }
}

// Backward of the rotation.  dBr_total[t] = dBr[t] + dBprev[t+1], dCr_total = dCr1 + dCr2.
//   d v = R(-theta) d out ;  d theta = -d out1 * out2 + d out2 * out1   (summed over B and C)
// dB / dC are summed over the heads of a group through shared memory (fixed order, deterministic).
template <class T>
__global__ void __launch_bounds__(256) rope_bwd_kernel(const T* __restrict__ B, const T* __restrict__ C,
                                                       const float* __restrict__ cum, const T* __restrict__ dBr,
                                                       const T* __restrict__ dBprev, const T* __restrict__ dCr1,
                                                       const T* __restrict__ dCr2, T* __restrict__ dB, T* __restrict__ dC,
                                                       float* __restrict__ dcum, int Tlen, int h, int g, int n) {
    extern __shared__ float sm[];  // [2][h][n]: d(un-rotated) B and C per head
    const int t = blockIdx.x, bb = blockIdx.y;
    const int half = n / 2, hpg = h / g;
    const size_t row = (size_t)bb * Tlen + t;
    float* sB = sm;
    float* sC = sm + (size_t)h * n;
    for (int e = threadIdx.x; e < h * half; e += 256) {
        const int hh = e / half, m = e - hh * half;
        const int gg = hh / hpg;
        float s, c;
        sincos_reduced(cum[row * h * half + e], &s, &c);
        const size_t ib = (row * g + gg) * n + m;
        const float b1 = to_f(B[ib]), b2 = to_f(B[ib + half]);
        const float c1 = to_f(C[ib]), c2 = to_f(C[ib + half]);
        const size_t o = (row * h + hh) * n + m;
        float db1 = to_f(dBr[o]), db2 = to_f(dBr[o + half]);
        if (t + 1 < Tlen) {
            db1 += to_f(dBprev[o + (size_t)h * n]);
            db2 += to_f(dBprev[o + (size_t)h * n + half]);
        }
        const float dc1 = to_f(dCr1[o]) + to_f(dCr2[o]), dc2 = to_f(dCr1[o + half]) + to_f(dCr2[o + half]);
        const float ob1 = b1 * c - b2 * s, ob2 = b1 * s + b2 * c;
        const float oc1 = c1 * c - c2 * s, oc2 = c1 * s + c2 * c;
        dcum[row * h * half + e] = (-db1 * ob2 + db2 * ob1) + (-dc1 * oc2 + dc2 * oc1);
        sB[hh * n + m] = c * db1 + s * db2;
        sB[hh * n + m + half] = -s * db1 + c * db2;
        sC[hh * n + m] = c * dc1 + s * dc2;
        sC[hh * n + m + half] = -s * dc1 + c * dc2;
    }
    __syncthreads();
    for (int e = threadIdx.x; e < g * n; e += 256) {
        const int gg = e / n, nn = e - gg * n;
        float ab = 0.f, ac = 0.f;
        for (int hl = 0; hl < hpg; ++hl) {
            ab += sB[(gg * hpg + hl) * n + nn];
            ac += sC[(gg * hpg + hl) * n + nn];
        }
        dB[(row * g + gg) * n + nn] = from_f<T>(ab);
        dC[(row * g + gg) * n + nn] = from_f<T>(ac);
    }
}

// ------------------------------------------------------------------------------------------
// Trapezoidal products.  One warp per (position, head): lanes over headdim.
// ------------------------------------------------------------------------------------------
template <class T>
__global__ void __launch_bounds__(256) xprod_fwd_kernel(const T* __restrict__ x, const float* __restrict__ dt,
                                                        const float* __restrict__ lam, const float* __restrict__ A_head,
                                                        T* __restrict__ xg, T* __restrict__ xb, float* __restrict__ dA,
                                                        int Tlen, int h, int p, size_t rows) {
    const size_t w = (size_t)blockIdx.x * 8 + (threadIdx.x >> 5);  // (b, t, h) flattened
    if (w >= rows) return;
    const int lane = threadIdx.x & 31;
    const int hh = (int)(w % h);
    const int t = (int)((w / h) % Tlen);
    const float d = dt[w], l = lam[w], a = d * A_head[hh];
    const float gam = l * d, bet = (1.f - l) * d * __expf(a);
    if (lane == 0) dA[w] = a;
    const T* xr = x + w * p;
    const T* xp = xr - (size_t)h * p;  // previous position, same head
    for (int pp = lane; pp < p; pp += 32) {
        xg[w * p + pp] = from_f<T>(to_f(xr[pp]) * gam);
        xb[w * p + pp] = from_f<T>(t > 0 ? to_f(xp[pp]) * bet : 0.f);
    }
}

// dx[t] = dxg[t] gamma[t] + dxb[t+1] beta[t+1] + D dy[t];  dgam = <dxg, x>,  dbet[t] = <dxb[t], x[t-1]>,  dyx = <dy, x>
template <class T>
__global__ void __launch_bounds__(256) xprod_bwd_kernel(const T* __restrict__ x, const T* __restrict__ dy,
                                                        const T* __restrict__ dxg, const T* __restrict__ dxb,
                                                        const float* __restrict__ dt, const float* __restrict__ lam,
                                                        const float* __restrict__ A_head, const float* __restrict__ D,
                                                        T* __restrict__ dx, float* __restrict__ dgam,
                                                        float* __restrict__ dbet, float* __restrict__ dyx, int Tlen, int h,
                                                        int p, size_t rows) {
    const size_t w = (size_t)blockIdx.x * 8 + (threadIdx.x >> 5);
    if (w >= rows) return;
    const int lane = threadIdx.x & 31;
    const int hh = (int)(w % h);
    const int t = (int)((w / h) % Tlen);
    const float d = dt[w], l = lam[w];
    const float gam = l * d;
    float bet_next = 0.f;
    if (t + 1 < Tlen) {
        const size_t wn = w + h;
        const float dn = dt[wn], ln = lam[wn];
        bet_next = (1.f - ln) * dn * __expf(dn * A_head[hh]);
    }
    const float Dh = D ? D[hh] : 0.f;
    float ag = 0.f, ab = 0.f, ay = 0.f;
    for (int pp = lane; pp < p; pp += 32) {
        const size_t o = w * p + pp;
        const float xv = to_f(x[o]), dyv = to_f(dy[o]), g1 = to_f(dxg[o]);
        float v = g1 * gam + Dh * dyv;
        if (t + 1 < Tlen) v += to_f(dxb[o + (size_t)h * p]) * bet_next;
        dx[o] = from_f<T>(v);
        ag += g1 * xv;
        ay += dyv * xv;
        if (t > 0) ab += to_f(dxb[o]) * to_f(x[o - (size_t)h * p]);
    }
#pragma unroll
    for (int of = 16; of > 0; of >>= 1) {
        ag += __shfl_xor_sync(0xffffffffu, ag, of);
        ab += __shfl_xor_sync(0xffffffffu, ab, of);
        ay += __shfl_xor_sync(0xffffffffu, ay, of);
    }
    if (lane == 0) {
        dgam[w] = ag;
        dbet[w] = ab;
        dyx[w] = ay;
    }
}

}  // namespace m3
}  // namespace ssd
