// Tile walk kernels of the tensor-core path (included by ssd_tc.cuh).
//
// One CTA per (batch, head) walks the 128-position tiles in order with the recurrent state
// (64 x 128, fp32) in registers.  Ten warps:
//   warps 0-7  "row" warps: thread (row = tid & 127, half = tid >> 7) owns TMEM lane `row` and one
//              half of the columns of every accumulator; they do the decay-mask epilogue, the output
//              epilogue and the state update;
//   warp 8     one lane issues every tcgen05.mma (the issuing lane is held about as long as the products take,
//              so it does nothing else);
//   warp 9     one lane issues every TMA load and store.
// Loads are multi-buffered (NST stages), the decay-masked C.B^T operand lives in TMEM (bf16 pairs,
// A operand of the next MMA), and S = C.B^T of tile k+1 is issued before the epilogue of tile k.
//
// mbarriers (phase = tile parity unless noted):
//   bar_ld[s]  TMA bytes of stage s landed                        (phase = (tile / NST) & 1)
//   bar_s      S = C.B^T of the tile is in TMEM                   (products -> row warps)
//   bar_u      weighted rows written, one arrival per warp         (row warps -> products)
//   bar_g      masked operand written (mode 0), one per warp       (row warps -> products)
//   bar_mh     Yo and Hl of the tile have completed: the state update runs while Yd does   (products -> row warps)
//   bar_m2     every MMA of the tile has completed                (products -> row warps, TMA lane: stage free)
//   bar_h      accumulators read, new state written, one per warp (row warps -> products, TMA lane)
//   bar_sr     the stores of the tile before have read sH / sY    (TMA lane -> products)
//
// MODE 0 forward (writes y), MODE 1 states only (stores the state entering every tile, bf16).  The reverse walk
// of the backward pass is rev_walk_kernel (ssd_tc_revwalk.cuh).
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

// MODE 0 exists in two instantiations (EXACT: diagonal mask blocks entry by entry, see kMaskSafeLog2); both are
// launched and the flag raised by tile_cumsum_kernel decides on the device which of the two does the work.  (As
// one kernel with two out-of-line bodies the walk was a quarter slower: the call boundary costs it registers.)
constexpr int kWalkThreads = 320;  // 8 row warps, the product-issue warp, the TMA warp

template <int MODE, bool EXACT = false>
__global__ void __launch_bounds__(kWalkThreads, 1) walk_kernel(const __grid_constant__ WalkParams P) {
    if (MODE == 0 && (P.extreme[0] != 0) != EXACT) return;
    using Cfg = WalkCfg<MODE>;
    constexpr int NST = Cfg::NST;
    extern __shared__ uint8_t smem_raw[];
    // 1024-byte alignment by an offset on the __shared__ array itself, so that every access below stays a
    // shared-memory instruction (a pointer rebuilt from an integer would be a generic-address access)
    uint8_t* sm = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    uint8_t* sStage = sm;                                  // per stage: V panels 0,1 | U | C panels 0,1
    uint8_t* sUd = sStage + (size_t)NST * Cfg::STAGE_BYTES;  // weighted copy of U
    uint8_t* sH = sUd + PANEL;                             // state, bf16, [n][p]
    uint8_t* sY = sH + PANEL;                              // y staging (mode 0 only)
    float* scum2 = reinterpret_cast<float*>(sH + PANEL + (MODE == 0 ? PANEL : 0));  // [2][128]
    float* sf = scum2 + 2 * LT;                            // [2][128] column factors dt_j 2^(cend - c_j)
    float* sdtc = sf + 2 * LT;                             // [2][128] dt_j (EXACT instantiation only)
    __shared__ uint64_t bar_ld[3], bar_s, bar_u, bar_g, bar_mh, bar_m2, bar_h, bar_sr;
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
        mbar_init(&bar_s, 1);
        mbar_init(&bar_u, 8);
        mbar_init(&bar_g, 8);
        mbar_init(&bar_mh, 1);
        mbar_init(&bar_m2, 1);
        mbar_init(&bar_h, 8);
        mbar_init(&bar_sr, 1);
        mbar_fence_init();
    }
    if (warp == 8) {
        tmem_alloc(&tmem_slot, 512);
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
    const uint32_t tm = tmem_slot;
    // S double-buffered [0,256), masked operand (bf16 pairs) [256,320), Yd [320,384), Yo [384,448), Hl [448,512)
    const uint32_t tG = tm + 256, tYd = tm + 320, tYo = tm + 384, tHl = tm + 448;

    auto state_row = [&](int it) {  // row of tile `it` of this walk in the [b*nt*h*128][64] state tensor
        return (int)((((size_t)bb * nt + it) * P.h + hh) * DN);
    };
    if (warp == 8) {
        // ------------------------------------------------------------------ product lane: every tcgen05.mma
        if (lane == 0) {
            // low descriptor words (see desc_lo): K-major operands have leading offset 16, MN-major ones the panel pitch
            const uint32_t hMN = desc_lo(smem_u32(sH), PANEL), udMN = desc_lo(smem_u32(sUd), PANEL);
            const uint32_t stK = desc_lo(smem_u32(sStage), 16), stMN = desc_lo(smem_u32(sStage), PANEL);
            constexpr uint32_t PU = PANEL >> 4, SU = Cfg::STAGE_BYTES >> 4;  // panel and stage pitch in 16-byte units
            auto offK = [](int kk) { return (uint32_t)(((kk >> 2) * (int)PANEL + (kk & 3) * 32) >> 4); };
            auto offMN = [](int kk) { return (uint32_t)(kk * 128); };
            auto issue_S = [&](int it) {  // S = C B^T of tile `it` into TMEM buffer it & 1
                const uint32_t vK = stK + (uint32_t)(it % NST) * SU, cK = vK + 3 * PU, tS = tm + (it & 1) * 128;
#pragma unroll
                for (int kk = 0; kk < 8; ++kk) mma_ss_lo(tS, cK + offK(kk), vK + offK(kk), kIdescS, kk > 0);
                mma_commit(&bar_s);
            };
            for (int it = 0; it < nt; ++it) {
                const int s = it % NST;
                const uint32_t ph = it & 1;
                mbar_wait(&bar_ld[s], (it / NST) & 1, &failed);
                const uint32_t vMN = stMN + (uint32_t)s * SU, uMN = vMN + 2 * PU, cK = stK + (uint32_t)s * SU + 3 * PU;
                if (MODE == 0 && it == 0) {
                    tc_fence_after();
                    issue_S(0);
                }
                if (it > 0) mbar_wait_spin(&bar_h, (it - 1) & 1, &failed);  // new state in sH, accumulators free
                tc_fence_after();
                if (MODE == 0) {
#pragma unroll
                    for (int kk = 0; kk < 8; ++kk)  // Yo = C H^T : A = C K-major, B = the running state in sH, [n][p] MN-major
                        mma_ss_lo(tYo, cK + offK(kk), hMN + offMN(kk), kIdescKM, kk > 0);
                }
                mbar_wait_spin(&bar_u, ph, &failed);
                tc_fence_after();
#pragma unroll
                for (int kk = 0; kk < 8; ++kk)  // Hl = V^T Ud : both MN-major, K = position
                    mma_ss_lo(tHl, vMN + offMN(kk), udMN + offMN(kk), kIdescMM, kk > 0);
                // the rows rewrite sH after bar_mh and sY after bar_m2: the stores of the tile before must have read them
                mbar_wait_spin(&bar_sr, ph, &failed);
                mma_commit(&bar_mh);  // Yo and Hl done: the state update may start while Yd runs
                if (MODE == 0) {
                    mbar_wait_spin(&bar_g, ph, &failed);
                    tc_fence_after();
#pragma unroll
                    for (int kk = 0; kk < 8; ++kk)  // Yd = G' x : A in TMEM (K = j), B = x [j][p] MN-major
                        mma_ts_lo(tYd, tG + kk * 8, uMN + offMN(kk), kIdescKM, kk > 0);
                }
                mma_commit(&bar_m2);
                if (MODE == 0 && it + 1 < nt) {
                    mbar_wait(&bar_ld[(it + 1) % NST], ((it + 1) / NST) & 1, &failed);
                    tc_fence_after();
                    issue_S(it + 1);
                }
            }
        }
        __syncwarp();
    } else if (warp == 9) {
        // ------------------------------------------------------------------ TMA lane: every load and store
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
                if (MODE == 0) {
                    tma_load_2d(st + 3 * PANEL, &P.mC, &bar_ld[s], gg * DN, grow);
                    tma_load_2d(st + 4 * PANEL, &P.mC, &bar_ld[s], gg * DN + 64, grow);
                }
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
                    if (MODE == 0) tma_store_2d(&P.mY, sY, hh * HP, bb * P.T + (it - 1) * LT);
                    if (P.save_states) tma_store_2d(&P.mS, sH, 0, state_row(it));
                    tma_store_commit();
                }
                tma_store_wait_read();
                mbar_arrive(&bar_sr);  // sH and sY may be rewritten
            }
            if (MODE == 0) {
                mbar_wait_spin(&bar_h, (nt - 1) & 1, &failed);
                tma_store_2d(&P.mY, sY, hh * HP, bb * P.T + (nt - 1) * LT);
                tma_store_commit();
            }
            tma_store_wait_all();
        }
        __syncwarp();
    } else {
        // ------------------------------------------------------------------ row warps
        const float* tcum = P.tcum + bh * P.T;
        const float* dtT = P.dtT ? P.dtT + bh * P.T : nullptr;
        const uint32_t lanes = lane_base(warp);
        const float Dhead = (MODE == 0 && P.D) ? P.D[hh] : 0.f;
        const float* skipT = (MODE == 0 && P.skipT) ? P.skipT + bh * P.T : nullptr;  // per-position skip instead of D
        const bool has_skip = MODE == 0 && (P.D || P.skipT);
        // per-tile scalars are fetched one tile ahead
        auto tile_of = [&](int it) { return it; };
        float c_n = tcum[(size_t)tile_of(0) * LT + row];
        float cend_n = tcum[(size_t)tile_of(0) * LT + (row | 31)];
        float dt_n = dtT ? dtT[(size_t)tile_of(0) * LT + row] : 1.f;
        float sk_n = skipT ? skipT[(size_t)tile_of(0) * LT + row] : Dhead;

        for (int it = 0; it < nt; ++it) {
            const int k = tile_of(it);
            const int s = it % NST, buf = it & 1;
            const uint32_t ph = it & 1;
            const float c_i = c_n, cend = cend_n, dtv = dt_n, Dh = sk_n;
            if (it + 1 < nt) {
                const size_t o = (size_t)tile_of(it + 1) * LT;
                c_n = tcum[o + row];
                cend_n = tcum[o + (row | 31)];
                dt_n = dtT ? dtT[o + row] : 1.f;
                if (skipT) sk_n = skipT[o + row];
            }
            if (hf == 0) {
                scum2[buf * LT + row] = c_i;
                sf[buf * LT + row] = dtv * exp2f(cend - c_i);
                if (EXACT) sdtc[buf * LT + row] = dtv;
            }
            mbar_wait(&bar_ld[s], (it / NST) & 1, &failed);
            named_barrier(1, 256);

            const float Sk = scum2[buf * LT + LT - 1];
            uint8_t* st = sStage + (size_t)s * Cfg::STAGE_BYTES;
            uint8_t* sU = st + 2 * PANEL;
            // this thread's half row of U: keep x for the D skip, write the weighted copy
            uint32_t xrow[16];
            {
                // the row weight as a bf16 pair: one packed multiply per two elements (the product is rounded to
                // bf16 for the MMA anyway; rounding the weight first costs at most one more ulp of bf16)
                const float w = exp2f(Sk - c_i) * dtv;
                const __nv_bfloat162 w2 = __float2bfloat162_rn(w);
#pragma unroll
                for (int ch = 0; ch < 4; ++ch) {
                    uint4 v = *reinterpret_cast<const uint4*>(sU + sw128(row, hf * 4 + ch));
                    uint32_t* u = reinterpret_cast<uint32_t*>(&v);
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        xrow[ch * 4 + q] = u[q];
                        __nv_bfloat162 r = __hmul2(*reinterpret_cast<__nv_bfloat162*>(&u[q]), w2);
                        u[q] = *reinterpret_cast<uint32_t*>(&r);
                    }
                    *reinterpret_cast<uint4*>(sUd + sw128(row, hf * 4 + ch)) = v;
                }
            }
            fence_async_smem();
            mbar_arrive_warp(&bar_u);
            if (MODE == 0) {
                mbar_wait(&bar_s, ph, &failed);
                tc_fence_after();
                const uint32_t tS = tm + (it & 1) * 128;
                const int rowblk = row & ~31;  // warp-uniform
                uint32_t packed[32];
#pragma unroll
                for (int blk = 0; blk < 2; ++blk) {
                    const int c0 = hf * 64 + blk * 32;
                    if (c0 > rowblk) {
#pragma unroll
                        for (int q = 0; q < 16; ++q) packed[blk * 16 + q] = 0u;
                    } else {
                        uint32_t r[32];
                        tmem_ld32(tS + lanes + c0, r);
                        // row factor relative to the block's last column: <= 1 below the diagonal block
                        const float rf = exp2f(c_i - scum2[buf * LT + c0 + 31]);
                        const float4* f4 = reinterpret_cast<const float4*>(sf + buf * LT + c0);
                        tmem_ld_wait();
                        const bool diag = (c0 == rowblk);
                        const float2* S2 = reinterpret_cast<const float2*>(r);
                        const float2* F2 = reinterpret_cast<const float2*>(f4);
                        const float2 rf2 = make_float2(rf, rf);
                        if (EXACT && diag) {
                            // inside the diagonal block the two factors are 2^(+-decay across the block); this
                            // instantiation runs when that leaves the fp32 range somewhere and evaluates the block
                            // entry by entry
                            const float2* C2 = reinterpret_cast<const float2*>(scum2 + buf * LT + c0);
                            const float2* T2 = reinterpret_cast<const float2*>(sdtc + buf * LT + c0);
#pragma unroll
                            for (int q2 = 0; q2 < 16; ++q2) {
                                const float2 cj = C2[q2], tj = T2[q2];
                                float2 l;
                                l.x = (c0 + 2 * q2 > row) ? 0.f : tj.x * exp2f(c_i - cj.x);
                                l.y = (c0 + 2 * q2 + 1 > row) ? 0.f : tj.y * exp2f(c_i - cj.y);
                                const float2 v = mul2(S2[q2], l);
                                packed[blk * 16 + q2] = pack_bf16(v.x, v.y);
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
                                packed[blk * 16 + q2] = pack_bf16(v.x, v.y);
                            }
                        }
                    }
                }
                tmem_st32(tG + lanes + hf * 32, packed);
                tmem_st_wait();
            }
            if (MODE == 0) {
                tc_fence_before();
                mbar_arrive_warp(&bar_g);
            }

            // the state update needs Hl only, which completes before Yd: it runs while the rows would wait for Yd
            mbar_wait(&bar_mh, ph, &failed);
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
            mbar_wait(&bar_m2, ph, &failed);

            tc_fence_after();
            if (MODE == 0) {
                uint32_t a[32], o[32];
                tmem_ld32(tYd + lanes + hf * 32, a);
                tmem_ld32(tYo + lanes + hf * 32, o);
                const float e = exp2f(c_i);
                tmem_ld_wait();
                float y[32];
                {
                    const float2* A2 = reinterpret_cast<const float2*>(a);
                    const float2* O2 = reinterpret_cast<const float2*>(o);
                    float2* Y2 = reinterpret_cast<float2*>(y);
                    const float2 e2 = make_float2(e, e), D2 = make_float2(Dh, Dh);
#pragma unroll
                    for (int q = 0; q < 16; ++q) {
                        float2 v = fma2(e2, O2[q], A2[q]);
                        if (has_skip) v = fma2(D2, __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&xrow[q])), v);
                        Y2[q] = v;
                    }
                }
                store_half_row(sY, row, hf * 4, y);
                if (P.ysq) {  // sum of squares of this half row, for the norm over all heads that follows the scan
                    float2 q2 = make_float2(0.f, 0.f);
                    const float2* Y2 = reinterpret_cast<const float2*>(y);
#pragma unroll
                    for (int q = 0; q < 16; ++q) q2 = fma2(Y2[q], Y2[q], q2);
                    P.ysq[((((size_t)bb * nt + k) * P.h + hh) * 2 + hf) * LT + row] = q2.x + q2.y;
                }
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
    if (warp == 8) tmem_dealloc(tm, 512);
}

}  // namespace tc
}  // namespace ssd
