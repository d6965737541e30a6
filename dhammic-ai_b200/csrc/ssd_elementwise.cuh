// The two element-wise operators that feed the scan in the reference's block, as stand-alone kernels:
//
//   rotation      y = rope(x, angles)            src/kernels/rope.py:39-193 (FusedRoPE), interleaved pairs
//                 (x[2m], x[2m+1]) -> (c x1 - s x2, s x1 + c x2); angles (B,T,1,D/2) broadcast over heads or
//                 (B,T,H,D/2) per head; backward dx = R(-a) dy, d a = dy_e (-s x1 - c x2) + dy_o (c x1 - s x2),
//                 summed over heads when the angles are broadcast.
//   coefficients  dt = softplus(dt_raw + dt_bias), lam = sigmoid(lam_raw), A = -exp(A_log), dA = dt A,
//                 beta = (1 - lam) dt exp(dA), gamma = lam dt        src/kernels/trapezoidal.py:89-214
//                 backward as derived there (:30-60), with the per-head sums of d dt_bias, d A_log reduced in a
//                 fixed order.
//
// Both are HBM-bound streaming kernels: 16-byte vector accesses on the wide tensors, fp32 arithmetic.
#pragma once
#include "ssd_common.cuh"
#include "ssd_mamba3.cuh"

namespace ssd {
namespace ew {

using m3::load_elems;
using m3::store_elems;
using m3::VecOf;

// ------------------------------------------------------------------------------------------
// Rotation.  One block per (b, t); a thread takes V consecutive elements (V/2 pairs) of one head.
// ------------------------------------------------------------------------------------------
template <class T, int V>
__global__ void __launch_bounds__(256) rope_op_fwd_kernel(const T* __restrict__ x, const float* __restrict__ ang,
                                                          T* __restrict__ y, int H, int D, int aH) {
    const size_t bt = blockIdx.x;
    const int half = D / 2, upr = D / V;
    for (int e = threadIdx.x; e < H * upr; e += 256) {
        const int hh = e / upr, j0 = (e - hh * upr) * V;
        float v[V], o[V];
        load_elems<T, V>(x + (bt * H + hh) * D + j0, v);
        const float* ap = ang + (bt * aH + (aH == 1 ? 0 : hh)) * half + j0 / 2;
#pragma unroll
        for (int q = 0; q < V / 2; ++q) {
            float s, c;
            sincosf(ap[q], &s, &c);
            o[2 * q] = c * v[2 * q] - s * v[2 * q + 1];
            o[2 * q + 1] = s * v[2 * q] + c * v[2 * q + 1];
        }
        store_elems<T, V>(y + (bt * H + hh) * D + j0, o);
    }
}

// One block per (b, t); a thread owns V/2 pair indices and walks the heads, so the sum over heads of the
// broadcast case stays in registers (fixed order).
template <class T, int V>
__global__ void __launch_bounds__(128) rope_op_bwd_kernel(const T* __restrict__ x, const float* __restrict__ ang,
                                                          const T* __restrict__ dy, T* __restrict__ dx,
                                                          float* __restrict__ dang, int H, int D, int aH) {
    const size_t bt = blockIdx.x;
    const int half = D / 2, upr = D / V;
    for (int u = threadIdx.x; u < upr; u += 128) {
        const int j0 = u * V;
        float acc[V / 2];
#pragma unroll
        for (int q = 0; q < V / 2; ++q) acc[q] = 0.f;
        float s[V / 2], c[V / 2];
        if (aH == 1) {
#pragma unroll
            for (int q = 0; q < V / 2; ++q) sincosf(ang[bt * half + j0 / 2 + q], &s[q], &c[q]);
        }
        for (int hh = 0; hh < H; ++hh) {
            if (aH != 1) {
#pragma unroll
                for (int q = 0; q < V / 2; ++q) sincosf(ang[(bt * H + hh) * half + j0 / 2 + q], &s[q], &c[q]);
            }
            float v[V], g[V], o[V];
            load_elems<T, V>(x + (bt * H + hh) * D + j0, v);
            load_elems<T, V>(dy + (bt * H + hh) * D + j0, g);
#pragma unroll
            for (int q = 0; q < V / 2; ++q) {
                const float x1 = v[2 * q], x2 = v[2 * q + 1], ge = g[2 * q], go = g[2 * q + 1];
                o[2 * q] = c[q] * ge + s[q] * go;
                o[2 * q + 1] = -s[q] * ge + c[q] * go;
                const float d = ge * (-s[q] * x1 - c[q] * x2) + go * (c[q] * x1 - s[q] * x2);
                if (aH == 1) acc[q] += d;
                else dang[(bt * H + hh) * half + j0 / 2 + q] = d;
            }
            store_elems<T, V>(dx + (bt * H + hh) * D + j0, o);
        }
        if (aH == 1) {
#pragma unroll
            for (int q = 0; q < V / 2; ++q) dang[bt * half + j0 / 2 + q] = acc[q];
        }
    }
}

// ------------------------------------------------------------------------------------------
// Coefficients.  Rows = all leading dimensions flattened, H columns; the parameters arrive as fp32 values
// already rounded to the working dtype (the reference casts them, src/kernels/trapezoidal.py:241-243).
// ------------------------------------------------------------------------------------------
__device__ __forceinline__ float softplus_f(float s) { return fmaxf(s, 0.f) + log1pf(__expf(-fabsf(s))); }
__device__ __forceinline__ float sigmoid_f(float s) { return 1.f / (1.f + __expf(-s)); }

template <class T>
__global__ void __launch_bounds__(256) trapezoid_fwd_kernel(const T* __restrict__ dt_raw, const T* __restrict__ lam_raw,
                                                            const float* __restrict__ dt_bias, const float* __restrict__ A_log,
                                                            T* __restrict__ dt, T* __restrict__ dA, T* __restrict__ beta,
                                                            T* __restrict__ gamma, size_t total, int H) {
    const size_t i = (size_t)blockIdx.x * 256 + threadIdx.x;
    if (i >= total) return;
    const int hh = (int)(i % H);
    const float d = softplus_f(to_f(dt_raw[i]) + dt_bias[hh]);
    const float l = sigmoid_f(to_f(lam_raw[i]));
    const float a = d * -expf(A_log[hh]);
    dt[i] = from_f<T>(d);
    dA[i] = from_f<T>(a);
    beta[i] = from_f<T>((1.f - l) * d * expf(a));
    gamma[i] = from_f<T>(l * d);
}

constexpr int TRAP_ROWS = 64;  // rows per block of the backward (one partial sum per block and head)

template <class T>
__global__ void __launch_bounds__(256) trapezoid_bwd_kernel(const T* __restrict__ dt_raw, const T* __restrict__ lam_raw,
                                                            const float* __restrict__ dt_bias, const float* __restrict__ A_log,
                                                            const T* __restrict__ g_dt, const T* __restrict__ g_dA,
                                                            const T* __restrict__ g_beta, const T* __restrict__ g_gamma,
                                                            T* __restrict__ d_dt_raw, T* __restrict__ d_lam_raw,
                                                            float* __restrict__ part_bias, float* __restrict__ part_alog,
                                                            size_t M, int H) {
    // thread = (row group, head column); a group walks every groups-th row of the block's TRAP_ROWS rows; the
    // group partials are then added in a fixed order
    __shared__ float sred[2][256];
    const size_t r0 = (size_t)blockIdx.x * TRAP_ROWS;
    const int cols = H < 256 ? H : 256, groups = 256 / cols;
    const int gi = threadIdx.x / cols, hc = threadIdx.x - gi * cols;
    for (int h0 = 0; h0 < H; h0 += cols) {
        const int hh = h0 + hc;
        float sb = 0.f, sa = 0.f;
        if (gi < groups && hh < H) {
            const float bias = dt_bias[hh], A = -expf(A_log[hh]);
            for (int r = gi; r < TRAP_ROWS && r0 + r < M; r += groups) {
                const size_t i = (r0 + r) * H + hh;
                const float s = to_f(dt_raw[i]) + bias;
                const float d = softplus_f(s), sig = sigmoid_f(s);
                const float l = sigmoid_f(to_f(lam_raw[i])), oml = 1.f - l;
                const float a = d * A, alpha = expf(a);
                const float gd = to_f(g_dt[i]), ga = to_f(g_dA[i]), gb = to_f(g_beta[i]), gg = to_f(g_gamma[i]);
                const float g_dt_total = gd + ga * A + gb * oml * alpha * (1.f + a) + gg * l;
                const float g_lam = -gb * d * alpha + gg * d;
                const float g_A = ga * d + gb * oml * d * d * alpha;
                const float g_raw = g_dt_total * sig;
                d_dt_raw[i] = from_f<T>(g_raw);
                d_lam_raw[i] = from_f<T>(g_lam * l * oml);
                sb += g_raw;
                sa += g_A * A;
            }
        }
        sred[0][threadIdx.x] = sb;
        sred[1][threadIdx.x] = sa;
        __syncthreads();
        if (gi == 0 && hh < H) {
            float tb = 0.f, ta = 0.f;
            for (int q = 0; q < groups; ++q) {
                tb += sred[0][q * cols + hc];
                ta += sred[1][q * cols + hc];
            }
            part_bias[(size_t)blockIdx.x * H + hh] = tb;
            part_alog[(size_t)blockIdx.x * H + hh] = ta;
        }
        __syncthreads();
    }
}

}  // namespace ew
}  // namespace ssd
