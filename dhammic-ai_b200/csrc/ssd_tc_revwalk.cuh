// Reverse tile walk of the backward pass (included by ssd_tc.cuh after ssd_tc_walk.cuh).
//
// One CTA per (batch, head) walks the 128-position tiles from the last to the first with the gradient of the
// recurrent state Q (128 x 64, fp32) in the registers of the eight row warps.  Per tile k it
//   * stores Q as it leaves tile k (bf16, [n][p]) for the per-tile backward kernel,
//   * writes exp(S_k) <Q, H_k> (the gradient of the decay between tiles; H_k = stored forward state),
//   * writes the state part of the decay gradient of every row, e_i * sum_p dY[i,p] (C_i . H_k[:,p]),
//   * updates Q <- exp(S_k) Q + C^T (e . dY).
// Only the last step is a recurrence, and it is a register update.  Everything else of tile k+1 (loads, the
// weighted rows, both MMAs) is independent of tile k, so the kernel is a software pipeline: three load stages,
// the two accumulators double-buffered in TMEM, and the row warps prepare tile k+1 while the MMAs of tile k
// run.  The weighted rows e_i * dY[i,:] are written in place over the loaded dY panel (each thread keeps its
// raw half row in registers for the row term).
//
// mbarriers (index = tile parity, phase = (tile / 2) & 1, unless noted):
//   bar_ld[s]  TMA bytes of stage s landed                         (index tile % 3, phase (tile / 3) & 1)
//   bar_u[b]   weighted rows of the tile written, 256 arrive        (row warps -> control)
//   bar_m[b]   both MMAs of the tile have completed                 (control -> row warps; frees the stage)
//   bar_a[b]   accumulators of the tile read, 256 arrive            (row warps -> control)
#pragma once

namespace ssd {
namespace tc {

constexpr int kRevStages = 3;
constexpr uint32_t kRevStageBytes = 4 * PANEL;  // C panels 0,1 | dY (weighted in place) | H_k
constexpr size_t kRevSmem = (size_t)kRevStages * kRevStageBytes + 2 * PANEL + 1024;  // stages | sQ[2] | alignment slack

__global__ void __launch_bounds__(288, 1) rev_walk_kernel(const __grid_constant__ WalkParams P) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* sStage = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    uint8_t* sQ = sStage + (size_t)kRevStages * kRevStageBytes;  // state gradient staged for its TMA store, bf16 [n][p], two buffers
    __shared__ uint64_t bar_ld[kRevStages], bar_u[2], bar_m[2], bar_a[2];
    __shared__ uint32_t tmem_slot;
    __shared__ int failed;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int hh = blockIdx.x, bb = blockIdx.y;
    const int gg = hh / P.hpg;
    const size_t bh = (size_t)bb * P.h + hh;
    const int nt = P.nt;

    if (tid == 0) {
        failed = 0;
        for (int s = 0; s < kRevStages; ++s) mbar_init(&bar_ld[s], 1);
        for (int b = 0; b < 2; ++b) {
            mbar_init(&bar_u[b], 256);
            mbar_init(&bar_m[b], 1);
            mbar_init(&bar_a[b], 256);
        }
        mbar_fence_init();
    }
    if (warp == 8) {
        tmem_alloc(&tmem_slot, 256);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tm = tmem_slot;  // Yo[2] at columns [0,128), Hl[2] at [128,256)

    if (warp == 8) {
        // ------------------------------------------------------------------ control lane
        if (lane == 0) {
            prefetch_tmap(&P.mU);
            prefetch_tmap(&P.mV);
            prefetch_tmap(&P.mC);
            auto issue_loads = [&](int it) {
                const int k = nt - 1 - it;
                const int s = it % kRevStages;
                uint8_t* st = sStage + (size_t)s * kRevStageBytes;
                const int grow = bb * P.T + k * LT;
                mbar_expect_tx(&bar_ld[s], kRevStageBytes);
                tma_load_2d(st, &P.mV, &bar_ld[s], gg * DN, grow);
                tma_load_2d(st + PANEL, &P.mV, &bar_ld[s], gg * DN + 64, grow);
                tma_load_2d(st + 2 * PANEL, &P.mU, &bar_ld[s], hh * HP, grow);
                tma_load_2d(st + 3 * PANEL, &P.mC, &bar_ld[s], 0, (int)((((size_t)bb * nt + k) * P.h + hh) * DN));
            };
            for (int it = 0; it < kRevStages && it < nt; ++it) issue_loads(it);
            for (int it = 0; it < nt; ++it) {
                const int s = it % kRevStages, b = it & 1;
                const uint32_t ph = (it >> 1) & 1;
                const uint32_t st = smem_u32(sStage + (size_t)s * kRevStageBytes);
                const uint32_t v0 = st, u0 = st + 2 * PANEL, h0 = st + 3 * PANEL;
                mbar_wait(&bar_ld[s], (it / kRevStages) & 1, &failed);
                if (it >= 2) mbar_wait(&bar_a[b], ((it - 2) >> 1) & 1, &failed);  // accumulators of tile it-2 read
                tc_fence_after();
#pragma unroll
                for (int kk = 0; kk < 8; ++kk) {  // Yo = C H_k : A = C K-major, B = H_k [n][p] MN-major
                    const uint32_t off = (kk >> 2) * PANEL + (kk & 3) * 32;
                    mma_ss(tm + b * 64, smem_desc(v0 + off, 16, 1024), smem_desc(h0 + kk * 2048, PANEL, 1024), kIdescKM, kk > 0);
                }
                mbar_wait(&bar_u[b], ph, &failed);
                tc_fence_after();
#pragma unroll
                for (int kk = 0; kk < 8; ++kk)  // Hl = C^T (e . dY) : both MN-major, K = position
                    mma_ss(tm + 128 + b * 64, smem_desc(v0 + kk * 2048, PANEL, 1024), smem_desc(u0 + kk * 2048, PANEL, 1024), kIdescMM, kk > 0);
                mma_commit(&bar_m[b]);
                // The stage of tile it-1 is free once its MMAs are done: the row warps read it for the last time
                // (H_k, for the decay term) before they arrived on bar_u of tile it, which was waited on above.
                if (it >= 1 && it + 2 < nt) {
                    mbar_wait(&bar_m[(it - 1) & 1], ((it - 1) >> 1) & 1, &failed);
                    issue_loads(it + 2);
                }
            }
        }
        __syncwarp();
    } else {
        // ------------------------------------------------------------------ row warps
        const int row = tid & 127, hf = tid >> 7;
        const float* tcum = P.tcum + bh * P.T;
        const uint32_t lanes = lane_base(warp);
        float H[32];  // state gradient row n = row, p in [hf*32, hf*32+32)
        if (P.seed) {
            const float* s = P.seed + bh * (size_t)HP * DN;
#pragma unroll
            for (int q = 0; q < 32; ++q) H[q] = s[(size_t)(hf * 32 + q) * DN + row];
        } else {
#pragma unroll
            for (int q = 0; q < 32; ++q) H[q] = 0.f;
        }
        // Store the state gradient leaving tile nt-1-it: staged in sQ[it & 1], written by one TMA store.  Thread 0
        // waits until the previous store (of the other buffer) has read its source before the barrier, so that
        // after the barrier every thread may overwrite that buffer one tile later.
        auto publish = [&](int it) {
            uint8_t* q = sQ + (size_t)(it & 1) * PANEL;
            store_half_row(q, row, hf * 4, H);
            if (tid == 0) tma_store_wait_read();
            fence_async_smem();
            named_barrier(1, 256);
            if (tid == 0) {
                tma_store_2d(&P.mS, q, 0, (int)((((size_t)bb * nt + (nt - 1 - it)) * P.h + hh) * DN));
                tma_store_commit();
            }
        };
        publish(0);

        uint32_t xrow[16], xnext[16];
        float c_i = 0.f, c_n = 0.f;
        // weighted copy of this thread's half row of dY of tile `it`, in place; the raw values stay in registers
        auto prepare = [&](int it, uint32_t (&keep)[16], float c) {
            const int s = it % kRevStages;
            mbar_wait(&bar_ld[s], (it / kRevStages) & 1, &failed);
            uint8_t* sU = sStage + (size_t)s * kRevStageBytes + 2 * PANEL;
            const __nv_bfloat162 w2 = __float2bfloat162_rn(exp2f(c));
#pragma unroll
            for (int ch = 0; ch < 4; ++ch) {
                uint4* p = reinterpret_cast<uint4*>(sU + sw128(row, hf * 4 + ch));
                uint4 v = *p;
                uint32_t* u = reinterpret_cast<uint32_t*>(&v);
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    keep[ch * 4 + q] = u[q];
                    __nv_bfloat162 r = __hmul2(*reinterpret_cast<__nv_bfloat162*>(&u[q]), w2);
                    u[q] = *reinterpret_cast<uint32_t*>(&r);
                }
                *p = v;
            }
            fence_async_smem();
            mbar_arrive(&bar_u[it & 1]);
        };
        c_i = tcum[(size_t)(nt - 1) * LT + row];
        float Sk = tcum[(size_t)(nt - 1) * LT + LT - 1];
        prepare(0, xrow, c_i);

        for (int it = 0; it < nt; ++it) {
            const int k = nt - 1 - it;
            const int s = it % kRevStages, b = it & 1;
            float Sk_n = 0.f;
            if (it + 1 < nt) {
                c_n = tcum[(size_t)(k - 1) * LT + row];
                Sk_n = tcum[(size_t)(k - 1) * LT + LT - 1];
            }
            const float dec = exp2f(Sk);
            {
                // exp(S_k) <Q, H_k>: Q is this thread's state row before the update of this tile, H_k the stored
                // forward state of the tile (rows n of the loaded panel)
                const uint8_t* sHk = sStage + (size_t)s * kRevStageBytes + 3 * PANEL;
                float q0 = 0.f, q1 = 0.f;
#pragma unroll
                for (int ch = 0; ch < 4; ++ch) {
                    uint4 hv = *reinterpret_cast<const uint4*>(sHk + sw128(row, hf * 4 + ch));
                    const uint32_t* hu = reinterpret_cast<const uint32_t*>(&hv);
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        float2 fh = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&hu[q]));
                        q0 = fmaf(fh.x, H[ch * 8 + 2 * q], q0);
                        q1 = fmaf(fh.y, H[ch * 8 + 2 * q + 1], q1);
                    }
                }
                float qh = (q0 + q1) * dec;
#pragma unroll
                for (int of = 16; of > 0; of >>= 1) qh += __shfl_xor_sync(0xffffffffu, qh, of);
                if (lane == 0) P.gS[((bh * (size_t)nt) + k) * 8 + warp] = qh;
            }
            if (it + 1 < nt) prepare(it + 1, xnext, c_n);

            mbar_wait(&bar_m[b], (it >> 1) & 1, &failed);
            tc_fence_after();
            uint32_t o[32], r[32];
            tmem_ld32(tm + b * 64 + lanes + hf * 32, o);
            tmem_ld32(tm + 128 + b * 64 + lanes + hf * 32, r);
            const float e = exp2f(c_i);
            tmem_ld_wait();
            tc_fence_before();
            mbar_arrive(&bar_a[b]);
            {
                // state part of the decay gradient of row i: e_i * sum_p dY[i,p] (C_i . H_k[:,p]); each half of the
                // row writes its own partial
                float a0 = 0.f, a1 = 0.f;
#pragma unroll
                for (int q = 0; q < 16; ++q) {
                    float2 f = __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&xrow[q]));
                    a0 = fmaf(__uint_as_float(o[2 * q]), f.x, a0);
                    a1 = fmaf(__uint_as_float(o[2 * q + 1]), f.y, a1);
                }
                P.rterm[((size_t)hf * gridDim.y * P.h + bh) * P.T + (size_t)k * LT + row] = e * (a0 + a1);
            }
            {
                float2* H2 = reinterpret_cast<float2*>(H);
                const float2 d2 = make_float2(dec, dec);
#pragma unroll
                for (int q = 0; q < 16; ++q) H2[q] = fma2(d2, H2[q], reinterpret_cast<const float2*>(r)[q]);
            }
            if (it + 1 < nt) publish(it + 1);
#pragma unroll
            for (int q = 0; q < 16; ++q) xrow[q] = xnext[q];
            c_i = c_n;
            Sk = Sk_n;
        }
        if (P.out_state) {
            float* o = P.out_state + bh * (size_t)HP * DN;
#pragma unroll
            for (int q = 0; q < 32; ++q) o[(size_t)(hf * 32 + q) * DN + row] = H[q];
        }
        if (tid == 0) tma_store_wait_all();
    }
    tc_fence_before();
    __syncthreads();
    if (tid == 0 && failed) atomicExch(P.status, 1);
    if (warp == 8) tmem_dealloc(tm, 256);
}

}  // namespace tc
}  // namespace ssd
