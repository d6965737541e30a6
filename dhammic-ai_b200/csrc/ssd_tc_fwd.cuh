// Forward walk of the tensor-core path (included by ssd_tc.cuh).
//
// One CTA per (batch, head) walks the 128-position tiles in order with the recurrent state (64 x 128, fp32) in
// registers.  Per tile k (V = B, U = x, C of the tile; H = state entering it; S_k = its total log2-decay):
//   S  = C V^T                     issued one tile ahead into a double-buffered TMEM accumulator
//   Yo = C H^T                     the entering state's part of the output
//   Hl = V^T (d dt o U)            the tile's contribution to the state; the weighted copy of U is made by the rows
//   G' = S o L o dt  (bf16 pairs, written back to TMEM by the rows),  Yd = G' U   (A operand from TMEM)
//   y  = e o Yo + Yd + skip o x,   H <- 2^{S_k} H + Hl
// 16 row warps: thread = (row, column quarter).  A quarter is one 32-column block of the causal mask (active iff
// quarter <= row block), 16 columns of every 64-wide accumulator and 16 values of the row's state.  (With two threads per
// row every per-tile step of a row thread was twice as long; the per-tile chain weighted copy -> mask -> Yd -> output is
// what bounds the kernel.)  A control warpgroup holds the lane that issues every tcgen05.mma and, in another warp, the
// lane that issues every TMA copy: the issuing lane of a product is held about as long as the product runs, so it
// does nothing else.  The kernel starts at 96 registers per thread; the control warpgroup gives registers back and the
// row warps take them (setmaxnreg).  Loads are double-buffered (80 KB per tile: the group's B and C panels and the
// head's x); the state update runs as soon as Hl is done, while Yd still runs.
//
// Shared memory: 2 stages of [V panels 0,1 | U | C panels 0,1] | weighted U | state (bf16 [n][p]) | y staging |
// per-column arrays.  TMEM: S double-buffered [0,256), G' [256,320), Yd [320,384), Yo [384,448), Hl [448,512).
//
// mbarriers (phase = tile parity unless noted):
//   bar_ld[s]  TMA bytes of stage s landed                        (phase = (tile / 2) & 1)
//   bar_s      S of the tile is in TMEM                           (products -> row warps)
//   bar_u      weighted rows written, one arrival per warp         (row warps -> products)
//   bar_g      masked operand written, one arrival per warp        (row warps -> products)
//   bar_mh     Yo and Hl of the tile have completed               (products -> row warps)
//   bar_m2     every product of the tile has completed            (products -> row warps, TMA lane: stage free)
//   bar_h      accumulators read, new state written, one per warp (row warps -> products, TMA lane)
//   bar_sr     the stores of the tile before have read sH / sY    (TMA lane -> products)
// The per-half-row sums of y^2 keep their (b, T/128, h, 2, 128) layout: the odd quarter of each half leaves its partial
// in shared memory, the even quarter adds its own and writes the sum after the block barrier at the top of the next tile.
//
// Two instantiations (EXACT: diagonal mask blocks entry by entry, see kMaskSafeLog2); both are launched and the flag
// raised by the cumulative-sum kernel decides on the device which of the two does the work.  (As one kernel with two
// out-of-line bodies the walk was a quarter slower: the call boundary costs it registers.)
#pragma once

namespace ssd {
namespace tc {

constexpr int kFwdThreads = 640;
constexpr int kFwdRegsLaunch = 96, kFwdRegsRow = 104, kFwdRegsCtl = 64;
static_assert(512 * kFwdRegsRow + 128 * kFwdRegsCtl <= kFwdThreads * kFwdRegsLaunch, "register trade exceeds the CTA's pool");
constexpr size_t kFwdSmem = WalkCfg<0>::SMEM + 4 * LT * 4;  // + partial sums of y^2 [2][2][128]

// 16 fp32 values of (row, quarter) as two 16-byte chunks of a 128-byte-swizzled [row][64] bf16 panel
__device__ __forceinline__ void store_quarter_row(uint8_t* panel, int row, int chunk0, const float (&v)[16]) {
#pragma unroll
    for (int ch = 0; ch < 2; ++ch) {
        uint4 o;
        o.x = pack_bf16(v[ch * 8 + 0], v[ch * 8 + 1]);
        o.y = pack_bf16(v[ch * 8 + 2], v[ch * 8 + 3]);
        o.z = pack_bf16(v[ch * 8 + 4], v[ch * 8 + 5]);
        o.w = pack_bf16(v[ch * 8 + 6], v[ch * 8 + 7]);
        *reinterpret_cast<uint4*>(panel + sw128(row, chunk0 + ch)) = o;
    }
}

template <bool EXACT>
__global__ void __maxnreg__(kFwdRegsLaunch) fwd_walk_kernel(const __grid_constant__ WalkParams P) {
    if ((P.extreme[0] != 0) != EXACT) return;
    using Cfg = WalkCfg<0>;
    constexpr int NST = Cfg::NST;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* sm = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    uint8_t* sStage = sm;                                  // per stage: V panels 0,1 | U | C panels 0,1
    uint8_t* sUd = sStage + (size_t)NST * Cfg::STAGE_BYTES;  // weighted copy of U
    uint8_t* sH = sUd + PANEL;                             // state, bf16, [n][p]
    uint8_t* sY = sH + PANEL;                              // y staging
    float* scum2 = reinterpret_cast<float*>(sY + PANEL);   // [2][128]
    float* sf = scum2 + 2 * LT;                            // [2][128] column factors dt_j 2^(cend - c_j)
    float* sdtc = sf + 2 * LT;                             // [2][128] dt_j (EXACT instantiation only)
    float* sysq = sdtc + 2 * LT;                           // [2][2][128] partial sums of y^2 of the odd quarters
    __shared__ uint64_t bar_ld[2], bar_s, bar_u, bar_g, bar_mh, bar_m2, bar_h, bar_sr;
    __shared__ uint32_t tmem_slot;
    __shared__ int failed;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int hh = blockIdx.x, bb = blockIdx.y;
    const int gg = hh / P.hpg;
    const size_t bh = (size_t)bb * P.h + hh;
    const int nt = P.nt;

    if (tid == 0) {
        failed = 0;
        mbar_init(&bar_ld[0], 1);
        mbar_init(&bar_ld[1], 1);
        mbar_init(&bar_s, 1);
        mbar_init(&bar_u, 16);
        mbar_init(&bar_g, 16);
        mbar_init(&bar_mh, 1);
        mbar_init(&bar_m2, 1);
        mbar_init(&bar_h, 16);
        mbar_init(&bar_sr, 1);
        mbar_fence_init();
    }
    if (warp == 16) {
        tmem_alloc(&tmem_slot, 512);
        tmem_relinquish();
    }
    const int row = tid & 127, q = (tid >> 7) & 3;
    // state row of this thread: n = row, p in [16 q, 16 q + 16)
    float H[16];
    if (warp < 16) {
        if (P.seed) {
            const float* s = P.seed + bh * (size_t)HP * DN;
#pragma unroll
            for (int j = 0; j < 16; ++j) H[j] = s[(size_t)(q * 16 + j) * DN + row];
        } else {
#pragma unroll
            for (int j = 0; j < 16; ++j) H[j] = 0.f;
        }
        store_quarter_row(sH, row, q * 2, H);
        fence_async_smem();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tm = tmem_slot;
    // S double-buffered [0,256), masked operand (bf16 pairs) [256,320), Yd [320,384), Yo [384,448), Hl [448,512)
    const uint32_t tG = tm + 256, tYd = tm + 320, tYo = tm + 384, tHl = tm + 448;
    auto state_row = [&](int it) {  // row of tile `it` of this walk in the [b*nt*h*128][64] state tensor
        return (int)((((size_t)bb * nt + it) * P.h + hh) * DN);
    };

    if (warp >= 16) {
        setmaxnreg_dec<kFwdRegsCtl>();
        if (warp == 16 && lane == 0) {
            // ------------------------------------------------------------------ product lane: every tcgen05.mma
            const uint32_t hMN = desc_lo(smem_u32(sH), PANEL), udMN = desc_lo(smem_u32(sUd), PANEL);
            const uint32_t stK = desc_lo(smem_u32(sStage), 16), stMN = desc_lo(smem_u32(sStage), PANEL);
            constexpr uint32_t PU = PANEL >> 4, SU = Cfg::STAGE_BYTES >> 4;  // panel and stage pitch in 16-byte units
            auto offK = [](int kk) { return (uint32_t)(((kk >> 2) * (int)PANEL + (kk & 3) * 32) >> 4); };
            auto offMN = [](int kk) { return (uint32_t)(kk * 128); };
            auto fresh = [](uint32_t v) {  // keeps the descriptors from being hoisted out of the tile loop (64 registers here)
                asm volatile("" : "+r"(v));
                return v;
            };
            auto issue_S = [&](int it) {  // S = C B^T of tile `it` into TMEM buffer it & 1
                const uint32_t vK = fresh(stK + (uint32_t)(it % NST) * SU), cK = vK + 3 * PU, tS = tm + (it & 1) * 128;
#pragma unroll
                for (int kk = 0; kk < 8; ++kk) mma_ss_lo(tS, cK + offK(kk), vK + offK(kk), kIdescS, kk > 0);
                mma_commit(&bar_s);
            };
            for (int it = 0; it < nt; ++it) {
                const int s = it % NST;
                const uint32_t ph = it & 1;
                mbar_wait(&bar_ld[s], (it / NST) & 1, &failed);
                const uint32_t vMN = fresh(stMN + (uint32_t)s * SU), uMN = vMN + 2 * PU, cK = fresh(stK + (uint32_t)s * SU + 3 * PU);
                const uint32_t hMN_ = fresh(hMN), udMN_ = fresh(udMN);
                if (it == 0) {
                    tc_fence_after();
                    issue_S(0);
                }
                if (it > 0) mbar_wait_spin(&bar_h, (it - 1) & 1, &failed);  // new state in sH, accumulators free
                tc_fence_after();
#pragma unroll
                for (int kk = 0; kk < 8; ++kk)  // Yo = C H^T : A = C K-major, B = the running state in sH, [n][p] MN-major
                    mma_ss_lo(tYo, cK + offK(kk), hMN_ + offMN(kk), kIdescKM, kk > 0);
                mbar_wait_spin(&bar_u, ph, &failed);
                tc_fence_after();
#pragma unroll
                for (int kk = 0; kk < 8; ++kk)  // Hl = V^T Ud : both MN-major, K = position
                    mma_ss_lo(tHl, vMN + offMN(kk), udMN_ + offMN(kk), kIdescMM, kk > 0);
                // the rows rewrite sH after bar_mh and sY after bar_m2: the stores of the tile before must have read them
                mbar_wait_spin(&bar_sr, ph, &failed);
                mma_commit(&bar_mh);  // Yo and Hl done: the state update may start while Yd runs
                mbar_wait_spin(&bar_g, ph, &failed);
                tc_fence_after();
#pragma unroll
                for (int kk = 0; kk < 8; ++kk)  // Yd = G' x : A in TMEM (K = j), B = x [j][p] MN-major
                    mma_ts_lo(tYd, tG + kk * 8, uMN + offMN(kk), kIdescKM, kk > 0);
                mma_commit(&bar_m2);
                if (it + 1 < nt) {
                    mbar_wait(&bar_ld[(it + 1) % NST], ((it + 1) / NST) & 1, &failed);
                    tc_fence_after();
                    issue_S(it + 1);
                }
            }
        } else if (warp == 17 && lane == 0) {
            // ------------------------------------------------------------------ TMA lane: every load and store
            prefetch_tmap(&P.mU);
            prefetch_tmap(&P.mV);
            prefetch_tmap(&P.mC);
            auto issue_loads = [&](int it) {
                const int s = it % NST;
                uint8_t* st = sStage + (size_t)s * Cfg::STAGE_BYTES;
                const int grow = bb * P.T + it * LT;
                mbar_expect_tx(&bar_ld[s], Cfg::STAGE_BYTES);
                tma_load_2d(st, &P.mV, &bar_ld[s], gg * DN, grow);
                tma_load_2d(st + PANEL, &P.mV, &bar_ld[s], gg * DN + 64, grow);
                tma_load_2d(st + 2 * PANEL, &P.mU, &bar_ld[s], hh * HP, grow);
                tma_load_2d(st + 3 * PANEL, &P.mC, &bar_ld[s], gg * DN, grow);
                tma_load_2d(st + 4 * PANEL, &P.mC, &bar_ld[s], gg * DN + 64, grow);
            };
            for (int it = 0; it < NST - 1 && it < nt; ++it) issue_loads(it);
            if (P.save_states) {  // the seed is the state entering the first tile
                tma_store_2d(&P.mS, sH, 0, state_row(0));
                tma_store_commit();
            }
            for (int it = 0; it < nt; ++it) {
                if (it + NST - 1 < nt) {
                    // the stage of tile it-1 is free once every product of that tile has completed
                    if (it > 0) mbar_wait(&bar_m2, (it - 1) & 1, &failed);
                    issue_loads(it + NST - 1);
                }
                if (it > 0) {
                    mbar_wait_spin(&bar_h, (it - 1) & 1, &failed);  // new state in sH, y staged
                    tma_store_2d(&P.mY, sY, hh * HP, bb * P.T + (it - 1) * LT);
                    if (P.save_states) tma_store_2d(&P.mS, sH, 0, state_row(it));
                    tma_store_commit();
                }
                tma_store_wait_read();
                mbar_arrive(&bar_sr);  // sH and sY may be rewritten
            }
            mbar_wait_spin(&bar_h, (nt - 1) & 1, &failed);
            tma_store_2d(&P.mY, sY, hh * HP, bb * P.T + (nt - 1) * LT);
            tma_store_commit();
            tma_store_wait_all();
        }
        __syncwarp();
    } else {
        // ------------------------------------------------------------------ row warps: thread = (row, column quarter)
        setmaxnreg_inc<kFwdRegsRow>();
        const int rb = row >> 5;  // row block, warp-uniform
        const bool active = q <= rb, diag = q == rb;
        const float* tcum = P.tcum + bh * P.T;
        const float* dtT = P.dtT ? P.dtT + bh * P.T : nullptr;
        const uint32_t lanes = lane_base(warp);
        const float Dhead = P.D ? P.D[hh] : 0.f;
        const float* skipT = P.skipT ? P.skipT + bh * P.T : nullptr;  // per-position skip instead of D
        const bool has_skip = P.D || P.skipT;
        const int c0 = q * 32;  // this thread's 32 columns of S
        // per-tile scalars are fetched one tile ahead
        float c_n = tcum[row];
        float cend_n = tcum[row | 31];
        float dt_n = dtT ? dtT[row] : 1.f;
        float sk_n = skipT ? skipT[row] : Dhead;
        float ysq_own = 0.f;  // even quarters: own partial of the tile before

        for (int it = 0; it < nt; ++it) {
            const int s = it % NST, buf = it & 1;
            const uint32_t ph = it & 1;
            const float c_i = c_n, cend = cend_n, dtv = dt_n, Dh = sk_n;
            if (it + 1 < nt) {
                const size_t o = (size_t)(it + 1) * LT;
                c_n = tcum[o + row];
                cend_n = tcum[o + (row | 31)];
                dt_n = dtT ? dtT[o + row] : 1.f;
                if (skipT) sk_n = skipT[o + row];
            }
            if (q == 0) {
                scum2[buf * LT + row] = c_i;
                sf[buf * LT + row] = dtv * exp2f(cend - c_i);
                if (EXACT) sdtc[buf * LT + row] = dtv;
            }
            mbar_wait(&bar_ld[s], (it / NST) & 1, &failed);
            named_barrier(1, 512);
            if (P.ysq && it > 0 && !(q & 1))  // the sum of the half row of the tile before: own quarter + the odd one's
                P.ysq[((((size_t)bb * nt + (it - 1)) * P.h + hh) * 2 + (q >> 1)) * LT + row] =
                    ysq_own + sysq[(((it - 1) & 1) * 2 + (q >> 1)) * LT + row];

            const float Sk = scum2[buf * LT + LT - 1];
            uint8_t* sU = sStage + (size_t)s * Cfg::STAGE_BYTES + 2 * PANEL;
            // this thread's quarter row of U: keep x for the skip term, write the weighted copy
            uint32_t xrow[8];
            {
                // the row weight as a bf16 pair: one packed multiply per two elements (the product is rounded to
                // bf16 for the MMA anyway; rounding the weight first costs at most one more ulp of bf16)
                const __nv_bfloat162 w2 = __float2bfloat162_rn(exp2f(Sk - c_i) * dtv);
#pragma unroll
                for (int ch = 0; ch < 2; ++ch) {
                    uint4 v = *reinterpret_cast<const uint4*>(sU + sw128(row, q * 2 + ch));
                    uint32_t* u = reinterpret_cast<uint32_t*>(&v);
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        xrow[ch * 4 + j] = u[j];
                        __nv_bfloat162 r = __hmul2(*reinterpret_cast<__nv_bfloat162*>(&u[j]), w2);
                        u[j] = *reinterpret_cast<uint32_t*>(&r);
                    }
                    *reinterpret_cast<uint4*>(sUd + sw128(row, q * 2 + ch)) = v;
                }
            }
            fence_async_smem();
            mbar_arrive_warp(&bar_u);

            mbar_wait(&bar_s, ph, &failed);
            tc_fence_after();
            {
                uint32_t packed[16];
                if (!active) {
#pragma unroll
                    for (int j = 0; j < 16; ++j) packed[j] = 0u;
                } else {
                    uint32_t r[32];
                    tmem_ld32(tm + (it & 1) * 128 + lanes + c0, r);
                    // row factor relative to the block's last column: <= 1 below the diagonal block
                    const float rf = exp2f(c_i - scum2[buf * LT + c0 + 31]);
                    const float2* F2 = reinterpret_cast<const float2*>(sf + buf * LT + c0);
                    tmem_ld_wait();
                    const float2* S2 = reinterpret_cast<const float2*>(r);
                    const float2 rf2 = make_float2(rf, rf);
                    if (EXACT && diag) {
                        // inside the diagonal block the two factors are 2^(+-decay across the block); this instantiation
                        // runs when that leaves the fp32 range somewhere and evaluates the block entry by entry
                        const float2* C2 = reinterpret_cast<const float2*>(scum2 + buf * LT + c0);
                        const float2* T2 = reinterpret_cast<const float2*>(sdtc + buf * LT + c0);
#pragma unroll
                        for (int q2 = 0; q2 < 16; ++q2) {
                            const float2 cj = C2[q2], tj = T2[q2];
                            float2 l;
                            l.x = (c0 + 2 * q2 > row) ? 0.f : tj.x * exp2f(c_i - cj.x);
                            l.y = (c0 + 2 * q2 + 1 > row) ? 0.f : tj.y * exp2f(c_i - cj.y);
                            const float2 v = mul2(S2[q2], l);
                            packed[q2] = pack_bf16(v.x, v.y);
                        }
                    } else {
#pragma unroll
                        for (int q2 = 0; q2 < 16; ++q2) {  // fp32 pairs: one instruction, two columns
                            float2 l = mul2(rf2, F2[q2]);
                            if (diag) {
                                if (c0 + 2 * q2 > row) l.x = 0.f;
                                if (c0 + 2 * q2 + 1 > row) l.y = 0.f;
                            }
                            const float2 v = mul2(S2[q2], l);
                            packed[q2] = pack_bf16(v.x, v.y);
                        }
                    }
                }
                tmem_st16(tG + lanes + q * 16, packed);
                tmem_st_wait();
            }
            tc_fence_before();
            mbar_arrive_warp(&bar_g);

            // the state update needs Hl only, which completes before Yd: it runs while the rows would wait for Yd
            mbar_wait(&bar_mh, ph, &failed);
            tc_fence_after();
            {
                uint32_t r[16];
                tmem_ld16(tHl + lanes + q * 16, r);
                const float dec = exp2f(Sk);
                tmem_ld_wait();
                float2* H2 = reinterpret_cast<float2*>(H);
                const float2 d2 = make_float2(dec, dec);
#pragma unroll
                for (int j = 0; j < 8; ++j) H2[j] = fma2(d2, H2[j], reinterpret_cast<const float2*>(r)[j]);
                store_quarter_row(sH, row, q * 2, H);
            }
            mbar_wait(&bar_m2, ph, &failed);
            tc_fence_after();
            {
                uint32_t a[16], o[16];
                tmem_ld16(tYd + lanes + q * 16, a);
                tmem_ld16(tYo + lanes + q * 16, o);
                const float e = exp2f(c_i);
                tmem_ld_wait();
                float y[16];
                const float2* A2 = reinterpret_cast<const float2*>(a);
                const float2* O2 = reinterpret_cast<const float2*>(o);
                float2* Y2 = reinterpret_cast<float2*>(y);
                const float2 e2 = make_float2(e, e), D2 = make_float2(Dh, Dh);
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    float2 v = fma2(e2, O2[j], A2[j]);
                    if (has_skip) v = fma2(D2, __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&xrow[j])), v);
                    Y2[j] = v;
                }
                store_quarter_row(sY, row, q * 2, y);
                if (P.ysq) {  // sum of squares of this quarter row, for the norm over all heads that follows the scan
                    float2 s2 = make_float2(0.f, 0.f);
#pragma unroll
                    for (int j = 0; j < 8; ++j) s2 = fma2(Y2[j], Y2[j], s2);
                    if (q & 1) sysq[((it & 1) * 2 + (q >> 1)) * LT + row] = s2.x + s2.y;
                    else ysq_own = s2.x + s2.y;
                }
            }
            tc_fence_before();
            fence_async_smem();
            mbar_arrive_warp(&bar_h);
        }
        if (P.ysq) {
            named_barrier(1, 512);
            if (!(q & 1))
                P.ysq[((((size_t)bb * nt + (nt - 1)) * P.h + hh) * 2 + (q >> 1)) * LT + row] =
                    ysq_own + sysq[(((nt - 1) & 1) * 2 + (q >> 1)) * LT + row];
        }
        if (P.out_state) {
            float* o = P.out_state + bh * (size_t)HP * DN;
#pragma unroll
            for (int j = 0; j < 16; ++j) o[(size_t)(q * 16 + j) * DN + row] = H[j];
        }
    }
    tc_fence_before();
    __syncthreads();
    if (tid == 0 && failed) atomicExch(P.status, 1);
    if (warp == 16) tmem_dealloc(tm, 512);
}

}  // namespace tc
}  // namespace ssd
