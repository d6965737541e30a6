// State walk of the tensor-core path and what the walk kernels share (included by ssd_tc.cuh).
//
// states_walk_kernel: one CTA per (batch, head) walks the 128-position tiles in order with the recurrent state
// (64 x 128, fp32) in registers and stores the state entering every tile as bf16 — the recurrence of the forward without
// its output.  The backward uses it when the forward did not keep the states.  Ten warps:
//   warps 0-7  "row" warps: thread (row = tid & 127, half = tid >> 7) owns TMEM lane `row` and one half of the
//              columns of the accumulator; they weight the rows of x and update the state;
//   warp 8     one lane issues every tcgen05.mma (the issuing lane is held about as long as the products take,
//              so it does nothing else);
//   warp 9     one lane issues every TMA load and store.
// The forward itself is fwd_walk_kernel (ssd_tc_fwd.cuh), the reverse walk of the backward rev_walk_kernel
// (ssd_tc_revwalk.cuh); WalkCfg<0> below is the shared-memory layout of the forward.
//
// mbarriers (phase = tile parity unless noted):
//   bar_ld[s]  TMA bytes of stage s landed                        (phase = (tile / NST) & 1)
//   bar_u      weighted rows written, one arrival per warp         (row warps -> products)
//   bar_m2     Hl of the tile has completed                       (products -> row warps, TMA lane: stage free)
//   bar_h      accumulator read, new state written, one per warp  (row warps -> products, TMA lane)
//   bar_sr     the store of the tile before has read sH           (TMA lane -> products)
#pragma once

namespace ssd {
namespace tc {

__device__ __forceinline__ void named_barrier(int id, int nthreads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}

// Write 32 fp32 values as bf16 into chunks [chunk0, chunk0+4) of this row of a swizzled panel.
__device__ __forceinline__ void store_half_row(uint8_t* panel, int row, int chunk0, const float (&v)[32]) {
#pragma unroll
    for (int ch = 0; ch < 4; ++ch) {
        uint4 o;
        o.x = pack_bf16(v[ch * 8 + 0], v[ch * 8 + 1]);
        o.y = pack_bf16(v[ch * 8 + 2], v[ch * 8 + 3]);
        o.z = pack_bf16(v[ch * 8 + 4], v[ch * 8 + 5]);
        o.w = pack_bf16(v[ch * 8 + 6], v[ch * 8 + 7]);
        *reinterpret_cast<uint4*>(panel + sw128(row, chunk0 + ch)) = o;
    }
}

// 32 fp32 state values of (row n, half hf) as 64 contiguous bytes of the [n][p] bf16 state tile `slot`.
__device__ __forceinline__ void store_state_slot(__nv_bfloat16* slot, int row, int hf, const float (&H)[32]) {
    uint4* o = reinterpret_cast<uint4*>(slot + (size_t)row * HP + hf * 32);
#pragma unroll
    for (int ch = 0; ch < 4; ++ch) {
        uint4 v;
        v.x = pack_bf16(H[ch * 8 + 0], H[ch * 8 + 1]);
        v.y = pack_bf16(H[ch * 8 + 2], H[ch * 8 + 3]);
        v.z = pack_bf16(H[ch * 8 + 4], H[ch * 8 + 5]);
        v.w = pack_bf16(H[ch * 8 + 6], H[ch * 8 + 7]);
        o[ch] = v;
    }
}

template <int MODE>
struct WalkCfg {
    static constexpr int NST = (MODE == 1) ? 3 : 2;              // load stages
    static constexpr int STAGE_PANELS = (MODE == 0) ? 5 : 3;                   // V(2) U(1) [C(2)]
    static constexpr uint32_t STAGE_BYTES = STAGE_PANELS * PANEL;
    // stages | sUd | sH | sY (mode 0) | scum2[2][128] sf[2][128] sdtc[2][128] | alignment slack
    static constexpr size_t SMEM = (size_t)NST * STAGE_BYTES + 2 * PANEL + (MODE == 0 ? PANEL : 0) + 6 * LT * 4 + 1024;
};

constexpr int kWalkThreads = 320;  // 8 row warps, the product-issue warp, the TMA warp

__global__ void __launch_bounds__(kWalkThreads, 1) states_walk_kernel(const __grid_constant__ WalkParams P) {
    using Cfg = WalkCfg<1>;
    constexpr int NST = Cfg::NST;
    extern __shared__ uint8_t smem_raw[];
    // 1024-byte alignment by an offset on the __shared__ array itself, so that every access below stays a
    // shared-memory instruction (a pointer rebuilt from an integer would be a generic-address access)
    uint8_t* sm = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    uint8_t* sStage = sm;                                  // per stage: V panels 0,1 | U
    uint8_t* sUd = sStage + (size_t)NST * Cfg::STAGE_BYTES;  // weighted copy of U
    uint8_t* sH = sUd + PANEL;                             // state, bf16, [n][p]
    __shared__ uint64_t bar_ld[3], bar_u, bar_m2, bar_h, bar_sr;
    __shared__ uint32_t tmem_slot;
    __shared__ int failed;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int hh = blockIdx.x, bb = blockIdx.y;
    const int gg = hh / P.hpg;
    const size_t bh = (size_t)bb * P.h + hh;
    const int nt = P.nt;

    if (tid == 0) {
        failed = 0;
        for (int s = 0; s < NST; ++s) mbar_init(&bar_ld[s], 1);
        mbar_init(&bar_u, 8);
        mbar_init(&bar_m2, 1);
        mbar_init(&bar_h, 8);
        mbar_init(&bar_sr, 1);
        mbar_fence_init();
    }
    if (warp == 8) {
        tmem_alloc(&tmem_slot, 64);
        tmem_relinquish();
    }
    const int row = tid & 127, hf = (tid >> 7) & 1;
    // state row of this thread: n = row, p in [hf*32, hf*32+32)
    float H[32];
    if (warp < 8) {
        if (P.seed) {
            const float* s = P.seed + bh * (size_t)HP * DN;
#pragma unroll
            for (int q = 0; q < 32; ++q) H[q] = s[(size_t)(hf * 32 + q) * DN + row];
        } else {
#pragma unroll
            for (int q = 0; q < 32; ++q) H[q] = 0.f;
        }
        store_half_row(sH, row, hf * 4, H);
        fence_async_smem();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tHl = tmem_slot;
    auto state_row = [&](int it) {  // row of tile `it` of this walk in the [b*nt*h*128][64] state tensor
        return (int)((((size_t)bb * nt + it) * P.h + hh) * DN);
    };
    if (warp == 8) {
        // ------------------------------------------------------------------ product lane
        if (lane == 0) {
            const uint32_t udMN = desc_lo(smem_u32(sUd), PANEL), stMN = desc_lo(smem_u32(sStage), PANEL);
            constexpr uint32_t SU = Cfg::STAGE_BYTES >> 4;  // stage pitch in 16-byte units
            for (int it = 0; it < nt; ++it) {
                const uint32_t ph = it & 1;
                const uint32_t vMN = stMN + (uint32_t)(it % NST) * SU;
                mbar_wait(&bar_ld[it % NST], (it / NST) & 1, &failed);
                if (it > 0) mbar_wait_spin(&bar_h, (it - 1) & 1, &failed);  // accumulator read
                mbar_wait_spin(&bar_u, ph, &failed);
                tc_fence_after();
#pragma unroll
                for (int kk = 0; kk < 8; ++kk)  // Hl = V^T Ud : both MN-major, K = position
                    mma_ss_lo(tHl, vMN + kk * 128, udMN + kk * 128, kIdescMM, kk > 0);
                // the rows rewrite sH after bar_m2: the store of the tile before must have read it
                mbar_wait_spin(&bar_sr, ph, &failed);
                mma_commit(&bar_m2);
            }
        }
        __syncwarp();
    } else if (warp == 9) {
        // ------------------------------------------------------------------ TMA lane
        if (lane == 0) {
            prefetch_tmap(&P.mU);
            prefetch_tmap(&P.mV);
            auto issue_loads = [&](int it) {
                const int s = it % NST;
                uint8_t* st = sStage + (size_t)s * Cfg::STAGE_BYTES;
                const int grow = bb * P.T + it * LT;
                mbar_expect_tx(&bar_ld[s], Cfg::STAGE_BYTES);
                tma_load_2d(st, &P.mV, &bar_ld[s], gg * DN, grow);
                tma_load_2d(st + PANEL, &P.mV, &bar_ld[s], gg * DN + 64, grow);
                tma_load_2d(st + 2 * PANEL, &P.mU, &bar_ld[s], hh * HP, grow);
            };
            for (int it = 0; it < NST - 1 && it < nt; ++it) issue_loads(it);
            tma_store_2d(&P.mS, sH, 0, state_row(0));  // the seed is the state entering the first tile
            tma_store_commit();
            for (int it = 0; it < nt; ++it) {
                if (it + NST - 1 < nt) {
                    // the stage of tile it-1 is free once the product of that tile has completed
                    if (it > 0) mbar_wait(&bar_m2, (it - 1) & 1, &failed);
                    issue_loads(it + NST - 1);
                }
                if (it > 0) {
                    mbar_wait_spin(&bar_h, (it - 1) & 1, &failed);  // new state in sH
                    tma_store_2d(&P.mS, sH, 0, state_row(it));
                    tma_store_commit();
                }
                tma_store_wait_read();
                mbar_arrive(&bar_sr);  // sH may be rewritten
            }
            tma_store_wait_all();
        }
        __syncwarp();
    } else {
        // ------------------------------------------------------------------ row warps
        const float* tcum = P.tcum + bh * P.T;
        const float* dtT = P.dtT ? P.dtT + bh * P.T : nullptr;
        const uint32_t lanes = lane_base(warp);
        // per-tile scalars are fetched one tile ahead
        float c_n = tcum[row], S_n = tcum[LT - 1];
        float dt_n = dtT ? dtT[row] : 1.f;
        for (int it = 0; it < nt; ++it) {
            const int s = it % NST;
            const uint32_t ph = it & 1;
            const float c_i = c_n, dtv = dt_n, Sk = S_n;
            if (it + 1 < nt) {
                const size_t o = (size_t)(it + 1) * LT;
                c_n = tcum[o + row];
                S_n = tcum[o + LT - 1];
                dt_n = dtT ? dtT[o + row] : 1.f;
            }
            mbar_wait(&bar_ld[s], (it / NST) & 1, &failed);
            {
                // (sUd is free: this thread waited for the product of the tile before, its only reader, before the state update)
                // this thread's half row of U, weighted by d_j dt_j as a bf16 pair (one packed multiply per two elements)
                const uint8_t* sU = sStage + (size_t)s * Cfg::STAGE_BYTES + 2 * PANEL;
                const __nv_bfloat162 w2 = __float2bfloat162_rn(exp2f(Sk - c_i) * dtv);
#pragma unroll
                for (int ch = 0; ch < 4; ++ch) {
                    uint4 v = *reinterpret_cast<const uint4*>(sU + sw128(row, hf * 4 + ch));
                    uint32_t* u = reinterpret_cast<uint32_t*>(&v);
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        __nv_bfloat162 r = __hmul2(*reinterpret_cast<__nv_bfloat162*>(&u[q]), w2);
                        u[q] = *reinterpret_cast<uint32_t*>(&r);
                    }
                    *reinterpret_cast<uint4*>(sUd + sw128(row, hf * 4 + ch)) = v;
                }
            }
            fence_async_smem();
            mbar_arrive_warp(&bar_u);
            mbar_wait(&bar_m2, ph, &failed);
            tc_fence_after();
            {
                uint32_t r[32];
                tmem_ld32(tHl + lanes + hf * 32, r);
                const float dec = exp2f(Sk);
                tmem_ld_wait();
#pragma unroll
                for (int q = 0; q < 16; ++q) {
                    float2* H2 = reinterpret_cast<float2*>(H);
                    H2[q] = fma2(make_float2(dec, dec), H2[q], reinterpret_cast<const float2*>(r)[q]);
                }
                store_half_row(sH, row, hf * 4, H);
            }
            tc_fence_before();
            fence_async_smem();
            mbar_arrive_warp(&bar_h);
        }
        if (P.out_state) {
            float* o = P.out_state + bh * (size_t)HP * DN;
#pragma unroll
            for (int q = 0; q < 32; ++q) o[(size_t)(hf * 32 + q) * DN + row] = H[q];
        }
    }
    tc_fence_before();
    __syncthreads();
    if (tid == 0 && failed) atomicExch(P.status, 1);
    if (warp == 8) tmem_dealloc(tHl, 64);
}

}  // namespace tc
}  // namespace ssd
