// The element-wise operators around the scan in the reference's block, as stand-alone kernels:
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
//   gate norm     out = rmsnorm(x, w) [* silu(z)]       src/kernels/rmsnorm.py:75-150, src/mamba_base_engine.py:189-191
//
// All are HBM-bound streaming kernels: 16-byte vector accesses on the wide tensors, fp32 arithmetic.
#pragma once
#include "ssd_common.cuh"
#include "ssd_mamba3.cuh"

namespace ssd {
namespace ew {

using m3::load_elems;
using m3::store_elems;
using m3::VecOf;

// V consecutive elements: one 16-byte vector, or a single element for V = 1
template <class T, int V>
__device__ __forceinline__ void load_elems1(const T* p, float (&f)[V]) {
    if constexpr (V == 1) f[0] = to_f(p[0]);
    else m3::load_vec<T, V>(p, f);
}
template <class T, int V>
__device__ __forceinline__ void store_elems1(T* p, const float (&f)[V]) {
    if constexpr (V == 1) p[0] = from_f<T>(f[0]);
    else m3::store_vec<T, V>(p, f);
}

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

// One block per (b, t); thread = (head slice, V/2 pair indices): it walks the heads of its slice, so the sum over
// heads of the broadcast case stays in registers per slice; the slices are then added in a fixed order through
// shared memory (deterministic).  With D / V pair groups per head, 128 / (D / V) slices share the heads.
template <class T, int V>
__global__ void __launch_bounds__(128) rope_op_bwd_kernel(const T* __restrict__ x, const float* __restrict__ ang,
                                                          const T* __restrict__ dy, T* __restrict__ dx,
                                                          float* __restrict__ dang, int H, int D, int aH) {
    __shared__ float sacc[128 * (V / 2)];
    const size_t bt = blockIdx.x;
    const int half = D / 2, upr = D / V;
    const int slices = upr >= 128 ? 1 : 128 / upr;
    const int sl = upr >= 128 ? 0 : threadIdx.x / upr;
    const int hps = (H + slices - 1) / slices;
    const int h_lo = sl * hps, h_hi = min(H, h_lo + hps);
    const int ustep = upr >= 128 ? 128 : upr;
    for (int u0 = 0; u0 < upr; u0 += ustep) {
        const int u = u0 + (upr >= 128 ? (int)threadIdx.x : (int)threadIdx.x - sl * upr);
        const bool live = sl < slices && u < upr;
        const int j0 = u * V;
        float acc[V / 2];
#pragma unroll
        for (int q = 0; q < V / 2; ++q) acc[q] = 0.f;
        if (live) {
            float s[V / 2], c[V / 2];
            if (aH == 1) {
#pragma unroll
                for (int q = 0; q < V / 2; ++q) sincosf(ang[bt * half + j0 / 2 + q], &s[q], &c[q]);
            }
            for (int hh = h_lo; hh < h_hi; ++hh) {
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
        }
        if (aH == 1) {  // block-uniform
            if (slices == 1) {
                if (live) {
#pragma unroll
                    for (int q = 0; q < V / 2; ++q) dang[bt * half + j0 / 2 + q] = acc[q];
                }
            } else {
                if (live) {
#pragma unroll
                    for (int q = 0; q < V / 2; ++q) sacc[(sl * upr + u) * (V / 2) + q] = acc[q];
                }
                __syncthreads();
                if (live && sl == 0) {
#pragma unroll
                    for (int q = 0; q < V / 2; ++q) {
                        float t = 0.f;
                        for (int k = 0; k < slices; ++k) t += sacc[(k * upr + u) * (V / 2) + q];
                        dang[bt * half + j0 / 2 + q] = t;
                    }
                }
                __syncthreads();
            }
        }
    }
}

// ------------------------------------------------------------------------------------------
// Coefficients.  Rows = all leading dimensions flattened, H columns; the parameters arrive as fp32 values
// already rounded to the working dtype (the reference casts them, src/kernels/trapezoidal.py:241-243).
// ------------------------------------------------------------------------------------------
__device__ __forceinline__ float softplus_f(float s) { return fmaxf(s, 0.f) + log1pf(__expf(-fabsf(s))); }
__device__ __forceinline__ float sigmoid_f(float s) { return __fdividef(1.f, 1.f + __expf(-s)); }

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


// ------------------------------------------------------------------------------------------
// RMS norm over the last dimension, optionally gated:  out = x * rsqrt(mean(x^2) + eps) * w  [* silu(z)]
// (src/kernels/rmsnorm.py:75-150; the block's closing `norm(y) * silu(z)`, src/mamba_base_engine.py:189-191).
// One warp per row, two passes over the row (the second one hits L1 / L2); V elements per lane and step.
//   backward:  dn = do [* silu(z)],  s = sum_j w_j x_j dn_j,  dx_i = r (w_i dn_i - x_i r^2 s / D),
//              dz_j = do_j n_j silu'(z_j),  dw_j = sum_rows x_j r dn_j  (a separate column reduction).
// ------------------------------------------------------------------------------------------
// V consecutive weights (16-byte vector loads when V is a multiple of 4: the column index then is too)
template <int V>
__device__ __forceinline__ void load_w(const float* __restrict__ p, float (&f)[V]) {
    if constexpr (V % 4 == 0) {
#pragma unroll
        for (int q = 0; q < V; q += 4) {
            const float4 v = *reinterpret_cast<const float4*>(p + q);
            f[q] = v.x; f[q + 1] = v.y; f[q + 2] = v.z; f[q + 3] = v.w;
        }
    } else {
#pragma unroll
        for (int q = 0; q < V; ++q) f[q] = p[q];
    }
}
__device__ __forceinline__ float silu_f(float z) { return z * sigmoid_f(z); }
__device__ __forceinline__ float silu_grad_f(float z) {
    const float sg = sigmoid_f(z);
    return sg * (1.f + z * (1.f - sg));
}

template <class T, int V>
__global__ void __launch_bounds__(256) rmsnorm_fwd_kernel(const T* __restrict__ x, const float* __restrict__ w,
                                                          const T* __restrict__ z, T* __restrict__ out,
                                                          float* __restrict__ rstd, size_t M, int D, float eps,
                                                          const float* __restrict__ ysq, int ysq_heads) {
    const size_t row = (size_t)blockIdx.x * 8 + (threadIdx.x >> 5);
    if (row >= M) return;
    const int lane = threadIdx.x & 31;
    const T* xr = x + row * D;
    float ss = 0.f;
    if (ysq) {
        // partial sums left by the scan's forward, [row / 128][head][half][row % 128]: the eight rows of a block are
        // neighbours, so the warps of the block share the sectors they read
        const float* pr = ysq + (row >> 7) * (size_t)(2 * ysq_heads) * 128 + (row & 127);
        for (int i = lane; i < 2 * ysq_heads; i += 32) ss += pr[(size_t)i * 128];
    } else {
#pragma unroll 4
        for (int c = lane * V; c < D; c += 32 * V) {
            float v[V];
            load_elems1<T, V>(xr + c, v);
#pragma unroll
            for (int q = 0; q < V; ++q) ss += v[q] * v[q];
        }
    }
#pragma unroll
    for (int of = 16; of > 0; of >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, of);
    const float r = rsqrtf(ss / (float)D + eps);
    if (lane == 0) rstd[row] = r;
#pragma unroll 4
    for (int c = lane * V; c < D; c += 32 * V) {
        float v[V], o[V], wv[V];
        load_elems1<T, V>(xr + c, v);
        load_w<V>(w + c, wv);
        if (z) {
            float g[V];
            load_elems1<T, V>(z + row * D + c, g);
#pragma unroll
            for (int q = 0; q < V; ++q) o[q] = v[q] * r * wv[q] * silu_f(g[q]);
        } else {
#pragma unroll
            for (int q = 0; q < V; ++q) o[q] = v[q] * r * wv[q];
        }
        store_elems1<T, V>(out + row * D + c, o);
    }
}

template <class T, int V>
__global__ void __launch_bounds__(256) rmsnorm_bwd_kernel(const T* __restrict__ x, const float* __restrict__ w,
                                                          const T* __restrict__ z, const T* __restrict__ dout,
                                                          const float* __restrict__ rstd, T* __restrict__ dx,
                                                          T* __restrict__ dz, size_t M, int D) {
    const size_t row = (size_t)blockIdx.x * 8 + (threadIdx.x >> 5);
    if (row >= M) return;
    const int lane = threadIdx.x & 31;
    const T* xr = x + row * D;
    const float r = rstd[row];
    float s = 0.f;
#pragma unroll 4
    for (int c = lane * V; c < D; c += 32 * V) {
        float v[V], g[V], wv[V];
        load_elems1<T, V>(xr + c, v);
        load_elems1<T, V>(dout + row * D + c, g);
        load_w<V>(w + c, wv);
        if (z) {
            float zz[V];
            load_elems1<T, V>(z + row * D + c, zz);
#pragma unroll
            for (int q = 0; q < V; ++q) g[q] *= silu_f(zz[q]);
        }
#pragma unroll
        for (int q = 0; q < V; ++q) s += wv[q] * v[q] * g[q];
    }
#pragma unroll
    for (int of = 16; of > 0; of >>= 1) s += __shfl_xor_sync(0xffffffffu, s, of);
    const float k = r * r * s / (float)D;
#pragma unroll 4
    for (int c = lane * V; c < D; c += 32 * V) {
        float v[V], g[V], o[V], wv[V];
        load_elems1<T, V>(xr + c, v);
        load_elems1<T, V>(dout + row * D + c, g);
        load_w<V>(w + c, wv);
        if (z) {
            float zz[V], oz[V];
            load_elems1<T, V>(z + row * D + c, zz);
#pragma unroll
            for (int q = 0; q < V; ++q) {
                oz[q] = g[q] * (v[q] * r * wv[q]) * silu_grad_f(zz[q]);
                g[q] *= silu_f(zz[q]);
            }
            store_elems1<T, V>(dz + row * D + c, oz);
        }
#pragma unroll
        for (int q = 0; q < V; ++q) o[q] = r * (wv[q] * g[q] - v[q] * k);
        store_elems1<T, V>(dx + row * D + c, o);
    }
}

// dw partials: block = 32 column threads (V columns each) x 8 row lanes over RMS_ROWS rows; the eight row lanes
// are added in a fixed order.
constexpr int RMS_ROWS = 256;
template <class T, int V>
__global__ void __launch_bounds__(256) rmsnorm_dw_kernel(const T* __restrict__ x, const T* __restrict__ z,
                                                         const T* __restrict__ dout, const float* __restrict__ rstd,
                                                         float* __restrict__ part, size_t M, int D) {
    __shared__ float sred[8][32 * V + 1];
    const int cl = threadIdx.x & 31, rl = threadIdx.x >> 5;
    const int col = (blockIdx.x * 32 + cl) * V;
    const size_t r0 = (size_t)blockIdx.y * RMS_ROWS;
    float acc[V];
#pragma unroll
    for (int q = 0; q < V; ++q) acc[q] = 0.f;
    if (col < D) {
#pragma unroll 4
        for (int r = rl; r < RMS_ROWS && r0 + r < M; r += 8) {
            const size_t i = (r0 + r) * D + col;
            float xv[V], g[V];
            load_elems1<T, V>(x + i, xv);
            load_elems1<T, V>(dout + i, g);
            if (z) {
                float zz[V];
                load_elems1<T, V>(z + i, zz);
#pragma unroll
                for (int q = 0; q < V; ++q) g[q] *= silu_f(zz[q]);
            }
            const float rr = rstd[r0 + r];
#pragma unroll
            for (int q = 0; q < V; ++q) acc[q] += xv[q] * rr * g[q];
        }
    }
#pragma unroll
    for (int q = 0; q < V; ++q) sred[rl][cl * V + q] = acc[q];
    __syncthreads();
    for (int e = threadIdx.x; e < 32 * V; e += 256) {
        const int c = blockIdx.x * 32 * V + e;
        if (c < D) {
            float t = 0.f;
#pragma unroll
            for (int q = 0; q < 8; ++q) t += sred[q][e];
            part[(size_t)blockIdx.y * D + c] = t;
        }
    }
}

}  // namespace ew
}  // namespace ssd
