// Reverse tile walk of the backward pass (included by ssd_tc.cuh after ssd_tc_walk.cuh).
//
// One CTA walks the 128-position tiles of NH heads of one group (same batch entry) from the last tile to the first,
// with the gradient of each head's recurrent state Q (128 x 64, fp32) in the registers of that head's eight row
// warps.  Per tile k and head it
//   * stores Q as it leaves tile k (bf16, [n][p]) for the per-tile backward kernel,
//   * updates Q <- exp(S_k) Q + C^T (e . dY).
// It reads dY and C only (the terms of the decay gradient that need the forward state are evaluated by the tile
// kernel, which has that state on chip anyway).  Only the update is a recurrence, and it is a register update;
// everything else of tile k+1 (loads, the weighted rows, the MMA) is independent of tile k, so the kernel is a
// software pipeline: three load stages, the accumulator double-buffered in TMEM, and the row warps prepare tile
// k+1 while the MMA of tile k runs.  The weighted rows e_i * dY[i,:] are written in place over the loaded dY panel.
// With NH = 2 the two heads share the C panels of a stage and one N = 128 product per tile
// (C^T [e dY_a | e dY_b]); their register chains are independent and run side by side on different warps.
//
// Threads: head hs = tid / 256 owns warps 8 hs .. 8 hs + 7 (thread = row, column half); the last warp issues TMA and MMA.
// mbarriers (index = tile parity, phase = (tile / 2) & 1, unless noted):
//   bar_ld[s]  TMA bytes of stage s landed                            (index tile % 3, phase (tile / 3) & 1)
//   bar_u[b]   weighted rows of the tile written, one arrival per warp (row warps -> control)
//   bar_m[b]   the MMA of the tile has completed                       (control -> row warps; frees the stage)
//   bar_a[b]   accumulator of the tile read, one arrival per warp     (row warps -> control)
#pragma once

namespace ssd {
namespace tc {

constexpr int kRevStages = 3;
template <int NH>
struct RevCfg {
    static constexpr uint32_t STAGE_BYTES = (2 + NH) * PANEL;  // C panels 0,1 | dY of each head (weighted in place)
    static constexpr size_t SMEM = (size_t)kRevStages * STAGE_BYTES + NH * PANEL + 128;  // stages | sQ per head | barriers
    static constexpr int THREADS = 256 * NH + 32;
};

template <int NH>
__global__ void __launch_bounds__(RevCfg<NH>::THREADS, 1) rev_walk_kernel(const __grid_constant__ WalkParams P) {
    using Cfg = RevCfg<NH>;
    // no static shared memory: the dynamic region starts at the CTA's shared-memory base
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t* sStage = smem_raw;
    uint8_t* sQ0 = sStage + (size_t)kRevStages * Cfg::STAGE_BYTES;  // per head: state gradient staged for its TMA store
    uint64_t* bars = reinterpret_cast<uint64_t*>(sQ0 + NH * PANEL);
    uint64_t* bar_ld = bars;          // [3]
    uint64_t* bar_u = bars + 3;       // [2]
    uint64_t* bar_m = bars + 5;       // [2]
    uint64_t* bar_a = bars + 7;       // [2]
    uint32_t& tmem_slot = *reinterpret_cast<uint32_t*>(bars + 9);
    int& failed = *reinterpret_cast<int*>(bars + 10);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (smem_u32(smem_raw) & 1023u) {  // the swizzled panels need a 1024-byte aligned base: report instead of computing garbage
        if (tid == 0) atomicExch(P.status, 2);
        return;
    }
    constexpr int CTLW = 8 * NH;  // control warp
    const int hh0 = blockIdx.x * NH, bb = blockIdx.y;
    const int gg = hh0 / P.hpg;
    const int nt = P.nt;

    if (tid == 0) {
        failed = 0;
        for (int s = 0; s < kRevStages; ++s) mbar_init(&bar_ld[s], 1);
        for (int b = 0; b < 2; ++b) {
            mbar_init(&bar_u[b], 8 * NH);
            mbar_init(&bar_m[b], 1);
            mbar_init(&bar_a[b], 8 * NH);
        }
        mbar_fence_init();
    }
    if (warp == CTLW) {
        tmem_alloc(&tmem_slot, 128 * NH);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tm = tmem_slot;  // accumulator of tile parity b at columns [b * 64 NH, (b + 1) * 64 NH), head hs at + 64 hs

    if (warp == CTLW) {
        // ------------------------------------------------------------------ control lane
        if (lane == 0) {
            prefetch_tmap(&P.mU);
            prefetch_tmap(&P.mV);
            auto issue_loads = [&](int it) {
                const int k = nt - 1 - it;
                const int s = it % kRevStages;
                uint8_t* st = sStage + (size_t)s * Cfg::STAGE_BYTES;
                const int grow = bb * P.T + k * LT;
                mbar_expect_tx(&bar_ld[s], Cfg::STAGE_BYTES);
                tma_load_2d(st, &P.mV, &bar_ld[s], gg * DN, grow);
                tma_load_2d(st + PANEL, &P.mV, &bar_ld[s], gg * DN + 64, grow);
#pragma unroll
                for (int hs = 0; hs < NH; ++hs) tma_load_2d(st + (2 + hs) * PANEL, &P.mU, &bar_ld[s], (hh0 + hs) * HP, grow);
            };
            for (int it = 0; it < kRevStages && it < nt; ++it) issue_loads(it);
            for (int it = 0; it < nt; ++it) {
                const int s = it % kRevStages, b = it & 1;
                const uint32_t ph = (it >> 1) & 1;
                const uint32_t st = smem_u32(sStage + (size_t)s * Cfg::STAGE_BYTES);
                const uint32_t v0 = st, u0 = st + 2 * PANEL;
                mbar_wait(&bar_ld[s], (it / kRevStages) & 1, &failed);
                if (it >= 2) mbar_wait(&bar_a[b], ((it - 2) >> 1) & 1, &failed);  // accumulator of tile it-2 read
                mbar_wait(&bar_u[b], ph, &failed);
                tc_fence_after();
#pragma unroll
                for (int kk = 0; kk < 8; ++kk)  // Hl = C^T [e . dY of each head] : both MN-major, K = position, N = 64 NH
                    mma_ss(tm + b * 64 * NH, smem_desc(v0 + kk * 2048, PANEL, 1024), smem_desc(u0 + kk * 2048, PANEL, 1024),
                           NH == 2 ? kIdescMM128 : kIdescMM, kk > 0);
                mma_commit(&bar_m[b]);
                // the stage of tile it-1 is free once its MMA is done
                if (it >= 1 && it - 1 + kRevStages < nt) {
                    mbar_wait(&bar_m[(it - 1) & 1], ((it - 1) >> 1) & 1, &failed);
                    issue_loads(it - 1 + kRevStages);
                }
            }
        }
        __syncwarp();
    } else {
        // ------------------------------------------------------------------ row warps
        const int hs = tid >> 8;  // which of the CTA's heads
        const int hh = hh0 + hs;
        const int ht = tid & 255, row = ht & 127, hf = ht >> 7;
        const size_t bh = (size_t)bb * P.h + hh;
        const float* tcum = P.tcum + bh * P.T;
        const uint32_t lanes = lane_base(warp);
        uint8_t* sQ = sQ0 + (size_t)hs * PANEL;
        float H[32];  // state gradient row n = row, p in [hf*32, hf*32+32)
        if (P.seed) {
            const float* s = P.seed + bh * (size_t)HP * DN;
#pragma unroll
            for (int q = 0; q < 32; ++q) H[q] = s[(size_t)(hf * 32 + q) * DN + row];
        } else {
#pragma unroll
            for (int q = 0; q < 32; ++q) H[q] = 0.f;
        }
        // Store the state gradient leaving tile nt-1-it: staged in the head's sQ panel, written by one TMA store of the
        // head's first thread, which waits until its previous store has read the panel; the first barrier (the head's
        // 256 threads) releases the panel to the writers, the second hands the written panel to the store.
        auto publish = [&](int it) {
            if (ht == 0) tma_store_wait_read();
            named_barrier(1 + 2 * hs, 256);
            store_half_row(sQ, row, hf * 4, H);
            fence_async_smem();
            named_barrier(2 + 2 * hs, 256);
            if (ht == 0) {
                tma_store_2d(&P.mS, sQ, 0, (int)((((size_t)bb * nt + (nt - 1 - it)) * P.h + hh) * DN));
                tma_store_commit();
            }
        };
        publish(0);

        float c_i = 0.f, c_n = 0.f;
        // weighted copy of this thread's half row of dY of tile `it`, in place
        auto prepare = [&](int it, float c) {
            const int s = it % kRevStages;
            mbar_wait(&bar_ld[s], (it / kRevStages) & 1, &failed);
            uint8_t* sU = sStage + (size_t)s * Cfg::STAGE_BYTES + (2 + hs) * PANEL;
            const __nv_bfloat162 w2 = __float2bfloat162_rn(exp2f(c));
#pragma unroll
            for (int ch = 0; ch < 4; ++ch) {
                uint4* p = reinterpret_cast<uint4*>(sU + sw128(row, hf * 4 + ch));
                uint4 v = *p;
                uint32_t* u = reinterpret_cast<uint32_t*>(&v);
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    __nv_bfloat162 r = __hmul2(*reinterpret_cast<__nv_bfloat162*>(&u[q]), w2);
                    u[q] = *reinterpret_cast<uint32_t*>(&r);
                }
                *p = v;
            }
            fence_async_smem();
            mbar_arrive_warp(&bar_u[it & 1]);
        };
        c_i = tcum[(size_t)(nt - 1) * LT + row];
        float Sk = tcum[(size_t)(nt - 1) * LT + LT - 1];
        prepare(0, c_i);

        for (int it = 0; it < nt; ++it) {
            const int k = nt - 1 - it;
            const int b = it & 1;
            float Sk_n = 0.f;
            if (it + 1 < nt) {
                c_n = tcum[(size_t)(k - 1) * LT + row];
                Sk_n = tcum[(size_t)(k - 1) * LT + LT - 1];
            }
            const float dec = exp2f(Sk);
            if (it + 1 < nt) prepare(it + 1, c_n);

            mbar_wait(&bar_m[b], (it >> 1) & 1, &failed);
            tc_fence_after();
            uint32_t r[32];
            tmem_ld32(tm + b * 64 * NH + hs * 64 + lanes + hf * 32, r);
            tmem_ld_wait();
            tc_fence_before();
            mbar_arrive_warp(&bar_a[b]);
            {
                float2* H2 = reinterpret_cast<float2*>(H);
                const float2 d2 = make_float2(dec, dec);
#pragma unroll
                for (int q = 0; q < 16; ++q) H2[q] = fma2(d2, H2[q], reinterpret_cast<const float2*>(r)[q]);
            }
            if (it + 1 < nt) publish(it + 1);
            c_i = c_n;
            Sk = Sk_n;
        }
        if (P.out_state) {
            float* o = P.out_state + bh * (size_t)HP * DN;
#pragma unroll
            for (int q = 0; q < 32; ++q) o[(size_t)(hf * 32 + q) * DN + row] = H[q];
        }
        if (ht == 0) tma_store_wait_all();
    }
    tc_fence_before();
    __syncthreads();
    if (tid == 0 && failed) atomicExch(P.status, 1);
    if (warp == CTLW) tmem_dealloc(tm, 128 * NH);
}

}  // namespace tc
}  // namespace ssd
