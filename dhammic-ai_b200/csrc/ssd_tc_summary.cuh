// Whole-sequence summaries of the tensor-core path (included by ssd_tc.cuh): what one contiguous piece of a
// sequence contributes to the state after it (forward) or to the gradient of the state before it (reverse),
// for a zero state on the other side.  These are the quantities the sequence-parallel schedule exchanges.
//
//   forward  F[n][p] = sum_j  B[j,n] * x[j,p] * dt_j * exp(sum of the log-decays AFTER position j)
//   reverse  D[n][p] = sum_i  C[i,n] * dy[i,p] *        exp(sum of the log-decays up to and including i)
//
// Neither is a recurrence: every tile adds one product to the same accumulator, so the kernel is a plain stream.
// One CTA per (batch entry, NH heads of a group): TMA loads (stages of the group's B or C panels + the x or dy panel of each
// head), eight warps per head scale the rows of their 64-wide panel in place, one lane issues eight tcgen05.mma per tile
// (N = 64 NH: the heads' panels side by side) that all accumulate into one TMEM accumulator, read once at the end.  With
// NH = 2 (heads per group even) the group's panels, two thirds of what a one-head CTA pulls in per tile, are fetched once
// for two heads; what one SM can pull in is what bounds this kernel.  The weights are <= 1 (dt aside), so nothing
// overflows; the forward walks the tiles from the last to the first (the decay after a tile is a running sum that starts
// at 0 where the weights are largest), the reverse from the first to the last.
//
// A given seed (initial state, or final-state gradient) enters as  exp(total log-decay) * seed.
// mbarriers, per stage s (phase (it / stages) & 1): bar_ld[s] TMA bytes landed; bar_u[s] rows scaled, one arrival per
// warp; bar_m[s] the products of the stage completed (the stage may be reloaded; the last one also releases the
// accumulator to the row warps).
#pragma once

namespace ssd {
namespace tc {

template <int NH>
struct SumCfg {
    static constexpr int STAGES = NH == 1 ? 4 : 3;
    static constexpr uint32_t STAGE_BYTES = (2 + NH) * PANEL;  // V panels 0,1 | U of each head
    static constexpr size_t SMEM = (size_t)STAGES * STAGE_BYTES + 1024;
    static constexpr int THREADS = 256 * NH + 32;
};

struct SummaryParams {
    CUtensorMap mU;        // x (forward) or dy (reverse): 2D [b*T][h*64]
    CUtensorMap mV;        // B (forward) or C (reverse):  2D [b*T][g*128]
    const float* tcum;     // (b,h,T) tile-cumulative log2-decay
    const float* dtT;      // (b,h,T) dt (forward) or null
    const float* seed;     // (b,h,p,n) fp32 or null
    float* out;            // (b,h,p,n) fp32
    float* logdecay;       // (b,h) total log-decay of the piece in natural-log units, or null
    int* status;
    int T, h, hpg, nt;
};

template <bool REV, int NH>
__global__ void __launch_bounds__(SumCfg<NH>::THREADS, 1) summary_kernel(const __grid_constant__ SummaryParams P) {
    using Cfg = SumCfg<NH>;
    constexpr int NS = Cfg::STAGES;
    constexpr int CTLW = 8 * NH;  // control warp
    extern __shared__ uint8_t smem_raw[];
    uint8_t* sStage = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    __shared__ uint64_t bar_ld[4], bar_u[4], bar_m[4];
    __shared__ uint32_t tmem_slot;
    __shared__ int failed;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int hh0 = blockIdx.x * NH, bb = blockIdx.y;
    const int gg = hh0 / P.hpg;
    const int nt = P.nt;
    // forward: tiles nt-1 .. 0; reverse: 0 .. nt-1
    auto tile_of = [&](int it) { return REV ? it : nt - 1 - it; };

    if (tid == 0) {
        failed = 0;
        for (int s = 0; s < NS; ++s) {
            mbar_init(&bar_ld[s], 1);
            mbar_init(&bar_u[s], 8 * NH);
            mbar_init(&bar_m[s], 1);
        }
        mbar_fence_init();
    }
    if (warp == CTLW) {
        tmem_alloc(&tmem_slot, 64 * NH);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tm = tmem_slot;  // accumulator row = n, columns [64 hs, 64 hs + 64) = p of head hs

    if (warp == CTLW) {
        if (lane == 0) {
            prefetch_tmap(&P.mU);
            prefetch_tmap(&P.mV);
            auto issue_loads = [&](int it) {
                const int s = it % NS;
                uint8_t* st = sStage + (size_t)s * Cfg::STAGE_BYTES;
                const int grow = bb * P.T + tile_of(it) * LT;
                mbar_expect_tx(&bar_ld[s], Cfg::STAGE_BYTES);
                tma_load_2d(st, &P.mV, &bar_ld[s], gg * DN, grow);
                tma_load_2d(st + PANEL, &P.mV, &bar_ld[s], gg * DN + 64, grow);
#pragma unroll
                for (int hs = 0; hs < NH; ++hs) tma_load_2d(st + (2 + hs) * PANEL, &P.mU, &bar_ld[s], (hh0 + hs) * HP, grow);
            };
            for (int it = 0; it < NS && it < nt; ++it) issue_loads(it);
            for (int it = 0; it < nt; ++it) {
                const int s = it % NS;
                const uint32_t st = smem_u32(sStage + (size_t)s * Cfg::STAGE_BYTES);
                mbar_wait(&bar_u[s], (it / NS) & 1, &failed);
                tc_fence_after();
#pragma unroll
                for (int kk = 0; kk < 8; ++kk)  // acc[n][p of every head] += V^T Uw : both MN-major, K = position
                    mma_ss(tm, smem_desc(st + kk * 2048, PANEL, 1024), smem_desc(st + 2 * PANEL + kk * 2048, PANEL, 1024),
                           NH == 2 ? kIdescMM128 : kIdescMM, it > 0 || kk > 0);
                mma_commit(&bar_m[s]);
                if (it >= 1 && it - 1 + NS < nt) {  // the stage of the tile before is free once its products are done
                    mbar_wait(&bar_m[(it - 1) % NS], ((it - 1) / NS) & 1, &failed);
                    issue_loads(it - 1 + NS);
                }
            }
        }
        __syncwarp();
    } else {
        const int hs = tid >> 8;  // which of the CTA's heads
        const int hh = hh0 + hs;
        const size_t bh = (size_t)bb * P.h + hh;
        const int ht = tid & 255, row = ht & 127, hf = ht >> 7;  // scaling: position `row`, columns [32 hf, 32 hf + 32) of the panel
        const float* tcum = P.tcum + bh * P.T;
        const float* dtT = (!REV && P.dtT) ? P.dtT + bh * P.T : nullptr;
        float run = 0.f;  // forward: log2-decay of the tiles after this one; reverse: of the tiles before it
        float c_n = tcum[(size_t)tile_of(0) * LT + row];
        float S_n = tcum[(size_t)tile_of(0) * LT + LT - 1];
        float dt_n = dtT ? dtT[(size_t)tile_of(0) * LT + row] : 1.f;
        for (int it = 0; it < nt; ++it) {
            const int s = it % NS;
            const float c_i = c_n, Sk = S_n, dtv = dt_n;
            if (it + 1 < nt) {
                const size_t o = (size_t)tile_of(it + 1) * LT;
                c_n = tcum[o + row];
                S_n = tcum[o + LT - 1];
                dt_n = dtT ? dtT[o + row] : 1.f;
            }
            const float w = REV ? exp2f(run + c_i) : dtv * exp2f(run + (Sk - c_i));
            run += Sk;
            mbar_wait(&bar_ld[s], (it / NS) & 1, &failed);
            uint8_t* sU = sStage + (size_t)s * Cfg::STAGE_BYTES + (2 + hs) * PANEL;
            const __nv_bfloat162 w2 = __float2bfloat162_rn(w);
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
            mbar_arrive_warp(&bar_u[s]);
        }
        // `run` is now the total log2-decay of the piece
        const int last = nt - 1;
        mbar_wait(&bar_m[last % NS], (last / NS) & 1, &failed);
        tc_fence_after();
        uint32_t r[32];
        tmem_ld32(tm + lane_base(warp) + hs * 64 + hf * 32, r);
        tmem_ld_wait();
        const float dec = exp2f(run);
        float* o = P.out + bh * (size_t)HP * DN;  // accumulator row = n, columns = p
        const float* sd = P.seed ? P.seed + bh * (size_t)HP * DN : nullptr;
#pragma unroll
        for (int q = 0; q < 32; ++q) {
            const size_t idx = (size_t)(hf * 32 + q) * DN + row;
            float v = __uint_as_float(r[q]);
            if (sd) v = fmaf(dec, sd[idx], v);
            o[idx] = v;
        }
        if (P.logdecay && ht == 0) P.logdecay[bh] = run * 0.6931471805599453f;
    }
    tc_fence_before();
    __syncthreads();
    if (tid == 0 && failed) atomicExch(P.status, 1);
    if (warp == CTLW) tmem_dealloc(tm, 64 * NH);
}

}  // namespace tc
}  // namespace ssd
