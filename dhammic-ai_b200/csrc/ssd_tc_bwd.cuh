// Tile-parallel backward kernel of the tensor-core path (included by ssd_tc.cuh).
//
// One CTA per (batch, 128-tile, group); the heads of the group run in an inner loop.  Per head h
// (X = x dt, L_ij = exp(cum_i - cum_j), d_j = exp(S - cum_j), e_i = exp(cum_i), H = state entering
// the tile, Q = gradient of the state leaving it; both stored by the walk kernels as bf16 [n][p]):
//
//   phase 1   S = C B^T,  dG = dY x^T                                     (TMEM, 2 x 128 columns)
//   mask      G = S o L (bf16 -> smem),  dS_h = dG o L o dt  (summed over heads in registers),
//             Xd = d dt x (in place in smem),  dYe = e dY (bf16 pairs -> TMEM)
//   phase 2   dX1 = G^T dY,  dX2 = B Q^T,  Yo = C H^T,  dC += dYe H,  dB += Xd Q   (dC, dB persist in TMEM)
//   rows      dx = dt (dX1 + d dX2) + D dy,  and the decay-gradient terms of the row, among them the two that
//             come from the state entering the tile: e_i <dY_i, Yo_i> for the row and exp(S) <Q, H> for the tile
// and once per group, after the heads:  dC += (sum_h dS_h) B,  dB += (sum_h dS_h)^T C.
//
// 16 row warps (thread = (row, column quarter)) and a control warpgroup of which two lanes work: one issues every
// tcgen05.mma, one every TMA copy.  The kernel is launched with 96 registers per thread; the control warpgroup gives
// registers back (setmaxnreg) and the row warps take them.  TMEM lanes are tied to warp % 4, so the rows 96-127, whose
// causal rows are the longest, can only be read by the warps of one SM sub-partition; four warps per 32-row block walk
// two 16-column steps each per head, and a quarter is exactly one 32-column block of the causal mask (active iff
// quarter <= row block, diagonal iff equal).  Per head:
//   rows     wait S, dG -> mask loop (G -> smem, dS summed over heads in registers) -> arrive A -> Xd = d dt x in place,
//            dYe = e dY -> TMEM -> arrive B -> <Q, H> from the shared panels while the products run -> Yo part of the
//            epilogue -> dX1, dX2 into registers -> arrive E -> dx staged, row sums -> arrive C -> block barrier of the
//            row warps (row sums of the four quarters added, next head's per-position scalars visible)
//   products A: Yo, dX1, dX2 -> B: dC, dB of the head -> E: S of the next head over dX1 / dX2 -> dC, dB done: dG of the
//            next head over Yo / dYe
//   copies   dC, dB done and E: H / Q of the next head, x / dy of the head after -> C: dx stored
// x / dy tiles are double-buffered across heads.  The per-position scalars of a head (tile-cumulative log2-decay, dt,
// skip coefficient) are fetched one head ahead into shared memory with asynchronous copies.  The per-row sums (gradient
// of the tile-cumulative log-decay, <dX, x>, <dy, x>) are summed over the four quarters in shared memory and leave
// the kernel as one array each.
//
// Two things measured while this was built, both about thread-to-thread mbarrier arrives: (1) an arrive that no later
// instruction depends on is scheduled after any amount of register-only work that follows it, so the row epilogue ties
// its first product to the arrive's token; (2) a lane that arrives for its warp does so with a predicated instruction,
// not a branch, so the warp stays converged.
#pragma once

namespace ssd {
namespace tc {

struct BwdParams {
    CUtensorMap mX, mdY, mB, mC;   // loads: [b*T][h*64] and [b*T][g*128]
    CUtensorMap mH, mQ;            // loads: states [b*nt*h*128][64]
    CUtensorMap mdX, mdB, mdC;     // stores
    const float* tcum;             // (b,h,T) tile-cumulative log2-decay
    const float* dtT;              // (b,h,T) or null
    const float* D;                // (h) or null
    const float* skipT;            // (b,h,T) per-position skip coefficient (replaces D), or null
    float* g;                      // (b,h,T) gradient w.r.t. the tile-cumulative log-decay
    float* ddtx;                   // (b,h,T) sum_p dX * x
    float* dyx;                    // (b,h,T) sum_p dy * x
    float* gS;                     // (b,h,nt,8): the terms that act through S = cum[127] of the tile
    const int* extreme;            // nonzero: the decay across some 32-position block is beyond the factorised mask
    int* status;
    int T, h, hpg, nt, b;
    int items;                     // nt * groups * b work items (tile, group, batch), tile fastest
};


// 13 operand panels | scum2, sfL, sdt, sD [2][128] | row partials [3][4][128] | warp partials [16] | alignment slack
constexpr size_t kBwdSmem = 13 * PANEL + 8 * LT * 4 + 12 * LT * 4 + 64 + 1024;
constexpr int kBwdThreads = 640;  // 16 row warps + the control warp's warpgroup (registers are budgeted per warpgroup)
// Registers per thread: at launch, and after the two warpgroup kinds have traded (setmaxnreg.inc waits for the pool, so the
// sum after the trade must not exceed what the CTA was launched with)
constexpr int kBwdRegsLaunch = 96, kBwdRegsRow = 104, kBwdRegsCtl = 64;
static_assert(512 * kBwdRegsRow + 128 * kBwdRegsCtl <= kBwdThreads * kBwdRegsLaunch, "register trade exceeds the CTA's pool");

// Two instantiations (EXACT: diagonal mask blocks entry by entry, see kMaskSafeLog2); both are launched and the
// extreme-decay flag decides on the device which of the two does the work (kept as separate kernels: as an
// out-of-line body this kernel loses registers to the call and spills).
template <bool EXACT>
__global__ void __maxnreg__(kBwdRegsLaunch) bwd_tile_kernel(const __grid_constant__ BwdParams P) {
    if ((P.extreme[0] != 0) != EXACT) return;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* sm = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    uint8_t* sC = sm;                  // 2 panels [pos][n]
    uint8_t* sB = sC + 2 * PANEL;      // 2 panels [pos][n]
    uint8_t* sG = sB + 2 * PANEL;      // 2 panels [i][j]; at the end dC staging
    uint8_t* sXY = sG + 2 * PANEL;     // 4 panels: x0, dy0, x1, dy1; at the end dB staging (2)
    uint8_t* sH = sXY + 4 * PANEL;     // [n][p]; at the end sum_h dS (with sQ)
    uint8_t* sQ = sH + PANEL;          // [n][p]
    uint8_t* sdX = sQ + PANEL;         // dx staging
    float* scum2 = reinterpret_cast<float*>(sdX + PANEL);  // [2][128] each:
    float* sfL = scum2 + 2 * LT;       //   2^(cend - c_j)
    float* sdt = sfL + 2 * LT;         //   dt_j
    float* sD = sdt + 2 * LT;          //   skip coefficient of the row (D of the head, or per position)
    float* sred = sD + 2 * LT;         // [3][4][128]: per-quarter partials of g, ddtx, dyx of the current head
    float* swred = sred + 12 * LT;     // [16]: per-warp partials of the S-borne term
    // TMA arrivals (count 1 + bytes): bar_cb, bar_xy[2], bar_hq.  Product completions (tcgen05.commit): bar_m1 (S, dG),
    // bar_m2 (dX1, dX2), bar_m2y (Yo), bar_m2b (dC, dB of the head), bar_m3 (group terms).  Row warps -> control (one arrival per warp):
    // bar_a (G staged), bar_b (Xd, dYe staged), bar_e (Yo, dX1, dX2 read), bar_c (dx staged),
    // bar_g1 (sum dS staged), bar_g2 (dC, dB staged).  TMA lane -> product lane: bar_sr (dx store has read its staging
    // panel), bar_sr2 (dC / dB stores have read theirs).
    __shared__ uint64_t bar_cb, bar_xy[2], bar_hq, bar_m1, bar_m2, bar_m2y, bar_m2b, bar_m3, bar_a, bar_b, bar_e, bar_c, bar_g1, bar_g2, bar_sr, bar_sr2;
    __shared__ uint32_t tmem_slot;
    __shared__ int failed;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    // Persistent over work items (tile k, group gg, batch bb).  `hc` counts heads and `ic` items since the start of
    // the kernel; every buffer index and mbarrier phase derives from them, in the row warps and in the control lanes alike.
    const int hpg = P.hpg, ngroups = P.h / P.hpg;
    const int item0 = blockIdx.x;
    const int k0 = item0 % P.nt, gg0 = (item0 / P.nt) % ngroups, bb0 = item0 / (P.nt * ngroups);

    if (tid == 0) {
        failed = 0;
        mbar_init(&bar_cb, 1);
        mbar_init(&bar_xy[0], 1);
        mbar_init(&bar_xy[1], 1);
        mbar_init(&bar_hq, 1);
        mbar_init(&bar_m1, 1);
        mbar_init(&bar_m2, 1);
        mbar_init(&bar_m2y, 1);
        mbar_init(&bar_m2b, 1);
        mbar_init(&bar_m3, 1);
        mbar_init(&bar_a, 16);
        mbar_init(&bar_b, 16);
        mbar_init(&bar_e, 16);
        mbar_init(&bar_c, 16);
        mbar_init(&bar_g1, 16);
        mbar_init(&bar_g2, 16);
        mbar_init(&bar_sr, 1);
        mbar_init(&bar_sr2, 1);
        mbar_fence_init();
    }
    if (warp == 1) {
        tmem_alloc(&tmem_slot, 512);
        tmem_relinquish();
    }
    const bool is_row = warp < 16;
    const int row = tid & 127, qc = (tid >> 7) & 3;  // column quarter: S / dG columns [32 qc, 32 qc + 32), p columns [16 qc, +16)
    // The per-position scalars of a head (tile-cumulative log2-decay, dt, skip coefficient) live in shared memory, two
    // buffers deep: the threads of column quarter 0 fetch those of the next head with asynchronous copies at the top of
    // a head and derive the per-column mask factor from them before the closing barrier of the row warps.
    auto fetch_scalars = [&](int buf, size_t o, int hh) {  // o: offset of the tile's first position in (b,h,T)
        cp_async4(&scum2[buf * LT + row], P.tcum + o + row);
        if (P.dtT) cp_async4(&sdt[buf * LT + row], P.dtT + o + row);
        if (P.skipT) cp_async4(&sD[buf * LT + row], P.skipT + o + row);
        else if (P.D) cp_async4(&sD[buf * LT + row], P.D + hh);
    };
    auto finish_scalars = [&](int buf) {  // all lanes of a quarter-0 warp
        cp_async_wait_all();
        __syncwarp();
        sfL[buf * LT + row] = exp2f(scum2[buf * LT + (row | 31)] - scum2[buf * LT + row]);
    };
    if (is_row && qc == 0) {
        sdt[row] = 1.f;
        sdt[LT + row] = 1.f;
        sD[row] = 0.f;
        sD[LT + row] = 0.f;
        __syncwarp();
        fetch_scalars(0, ((size_t)bb0 * P.h + gg0 * hpg) * P.T + (size_t)k0 * LT, gg0 * hpg);
        finish_scalars(0);
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tm = tmem_slot;
    // phase 1: S [0,128) dG [128,256).  Phase 2: dX1 [0,64) and dX2 [64,128) take the S columns, Yo = C H^T the dG
    // columns [160,224) and dYe (bf16 pairs) the dG columns [224,256), which only the rows 96-127 read in the mask
    // loop; persistent over heads: dC [256,384) dB [384,512)
    const uint32_t tS = tm, tdG = tm + 128, tX1 = tm, tX2 = tm + 64, tYo = tm + 160, tYe = tm + 224, tdC = tm + 256, tdB = tm + 384;

  if (!is_row) {
    // ======================= control warps: one lane issues every tcgen05.mma, one lane of the next warp every TMA copy.
    // Both derive the same sequence of items and heads; they meet only through the mbarriers.
    setmaxnreg_dec<kBwdRegsCtl>();
    if (warp == 16 && lane == 0) {
        // ---------------- product issue
        // Low descriptor words of the operands that stay put (K-major: leading offset 16; MN-major: the panel pitch);
        // the descriptor of K step kk adds offK(kk) or offMN(kk).
        const uint32_t cK = desc_lo(smem_u32(sC), 16), cMN = desc_lo(smem_u32(sC), PANEL);
        const uint32_t bK = desc_lo(smem_u32(sB), 16), bMN = desc_lo(smem_u32(sB), PANEL);
        const uint32_t gMN = desc_lo(smem_u32(sG), PANEL);
        const uint32_t hK = desc_lo(smem_u32(sH), 16), hMN = desc_lo(smem_u32(sH), PANEL);
        const uint32_t qK = desc_lo(smem_u32(sQ), 16), qMN = desc_lo(smem_u32(sQ), PANEL);
        const uint32_t xyK = desc_lo(smem_u32(sXY), 16);  // x of buffer 0; dy +PANEL, buffer 1 +2 PANEL (in 16-byte units)
        auto offK = [](int kk) { return (uint32_t)(((kk >> 2) * (int)PANEL + (kk & 3) * 32) >> 4); };  // two 64-wide panels
        auto offMN = [](int kk) { return (uint32_t)(kk * 128); };                                       // 2048 bytes per step
        constexpr uint32_t PU = PANEL >> 4;
        // The base words pass through an empty asm before each group of products, so that the compiler adds the step
        // offsets where they are used instead of keeping some eighty descriptors live across the loops (and spilling).
        auto fresh = [](uint32_t v) {
            asm volatile("" : "+r"(v));
            return v;
        };
        auto issue_S = [&]() {  // S = C B^T (K = n), the same for every head of the item
            const uint32_t c = fresh(cK), b = fresh(bK);
#pragma unroll
            for (int kk = 0; kk < 8; ++kk) mma_ss_lo(tS, c + offK(kk), b + offK(kk), kIdescKK128, kk > 0);
        };
        auto issue_dG = [&](uint32_t hcur) {  // dG = dY x^T (K = p) of the head with running index hcur
            const uint32_t x0 = fresh(xyK + 2 * PU * (hcur & 1)), y0 = x0 + PU;
#pragma unroll
            for (int kk = 0; kk < 4; ++kk) mma_ss_lo(tdG, y0 + 2 * kk, x0 + 2 * kk, kIdescKK128, kk > 0);
        };
        int item = item0;
        uint32_t hc = 0, ic = 0;
        mbar_wait(&bar_cb, 0, &failed);
        mbar_wait(&bar_xy[0], 0, &failed);
        tc_fence_after();
        issue_S();
        issue_dG(0);
        mma_commit(&bar_m1);
        for (;;) {
            const bool more = item + (int)gridDim.x < P.items;
            for (int hl = 0; hl < hpg; ++hl) {
                const uint32_t hcur = hc + hl;
                const int xb = hcur & 1;
                const uint32_t ph = hcur & 1;
                const uint32_t x0 = fresh(xyK + 2 * PU * xb);    // x (Xd) of this head, K-major
                const uint32_t yMN = x0 + PU + ((PANEL >> 4) << 16) - (1u << 16);  // dy of this head, MN-major
                const uint32_t cK_ = fresh(cK), bK_ = fresh(bK), gMN_ = fresh(gMN), hK_ = fresh(hK), hMN_ = fresh(hMN),
                               qK_ = fresh(qK), qMN_ = fresh(qMN);
                mbar_wait(&bar_hq, ph, &failed);  // H and Q of this head have landed
                mbar_wait_spin(&bar_a, ph, &failed);   // G complete, S and dG read by every row
                tc_fence_after();
#pragma unroll
                for (int kk = 0; kk < 8; ++kk)  // Yo = C H^T : A = C K-major (K = n), B = H^T [n][p] MN-major
                    mma_ss_lo(tYo, cK_ + offK(kk), hMN_ + offMN(kk), kIdescKM, kk > 0);
                mma_commit(&bar_m2y);  // the row epilogue starts on Yo ...
#pragma unroll
                for (int kk = 0; kk < 8; ++kk)  // dX1 = G^T dY : A = G MN-major (M = j, K = i), B = dY MN-major
                    mma_ss_lo(tX1, gMN_ + offMN(kk), yMN + offMN(kk), kIdescMM, kk > 0);
#pragma unroll
                for (int kk = 0; kk < 8; ++kk)  // dX2 = B Q^T : A = B K-major (K = n), B = Q^T [n][p] MN-major
                    mma_ss_lo(tX2, bK_ + offK(kk), qMN_ + offMN(kk), kIdescKM, kk > 0);
                // the rows write the dx staging panel after bar_m2: the store of the head before must have read it
                if (hcur > 0) mbar_wait_spin(&bar_sr, (hcur - 1) & 1, &failed);
                mma_commit(&bar_m2);  // ... and goes on with dX1 and dX2
                mbar_wait_spin(&bar_b, ph, &failed);  // Xd, dYe complete
                tc_fence_after();
#pragma unroll
                for (int kk = 0; kk < 4; ++kk)  // dC += dYe H : A in TMEM (K = p), B = H^T [n][p] K-major, N = 128
                    mma_ts_lo(tdC, tYe + kk * 8, hK_ + 2 * kk, kIdescKK128, hl > 0 || kk > 0);
#pragma unroll
                for (int kk = 0; kk < 4; ++kk)  // dB += Xd Q : A = Xd K-major (in place of x), B = Q^T [n][p] K-major
                    mma_ss_lo(tdB, x0 + 2 * kk, qK_ + 2 * kk, kIdescKK128, hl > 0 || kk > 0);
                mma_commit(&bar_m2b);  // releases H, Q, Xd and the dYe columns
                if (hl + 1 < hpg) {
                    // every row has read Yo, dX1 and dX2, and the dC / dB products have consumed dYe: the accumulators of
                    // this head are free, S and dG of the next head run while the rows finish their epilogue
                    mbar_wait_spin(&bar_e, ph, &failed);
                    tc_fence_after();
                    issue_S();  // over dX1 / dX2
                    mbar_wait(&bar_m2b, ph, &failed);
                    mbar_wait(&bar_xy[xb ^ 1], ((hcur + 1) >> 1) & 1, &failed);  // prefetched during this head
                    tc_fence_after();
                    issue_dG(hcur + 1);  // over Yo and dYe
                    mma_commit(&bar_m1);
                }
            }
            // ---- group terms
            mbar_wait_spin(&bar_g1, ic & 1, &failed);  // sum_h dS staged as bf16 [i][j] in the H / Q panels
            tc_fence_after();
            const uint32_t hK_ = fresh(hK), hMN_ = fresh(hMN), bMN_ = fresh(bMN), cMN_ = fresh(cMN);
#pragma unroll
            for (int kk = 0; kk < 8; ++kk)  // dC += dS B : A = dS K-major (K = j), B = B [j][n] MN-major, N = 128
                mma_ss_lo<true>(tdC, hK_ + offK(kk), bMN_ + offMN(kk), kIdescKM128);
#pragma unroll
            for (int kk = 0; kk < 8; ++kk)  // dB += dS^T C : A = dS MN-major (M = j, K = i), B = C [i][n] MN-major
                mma_ss_lo<true>(tdB, hMN_ + offMN(kk), cMN_ + offMN(kk), kIdescMM128);
            mma_commit(&bar_m3);
            if (!more) break;
            const uint32_t ic_done = ic;
            item += (int)gridDim.x;
            hc += hpg;
            ic += 1;
            // S and dG of the next item's first head run while the stores read their staging panels
            mbar_wait(&bar_cb, ic & 1, &failed);
            mbar_wait(&bar_xy[hc & 1], (hc >> 1) & 1, &failed);
            mbar_wait(&bar_m3, ic_done & 1, &failed);  // (the rows read dC / dB after this; S and dG live elsewhere)
            tc_fence_after();
            issue_S();
            issue_dG(hc);
            // S and dG are announced when the stores of dC and dB have read their staging panels: the rows overwrite
            // the G panels right after bar_m1
            mbar_wait_spin(&bar_sr2, ic_done & 1, &failed);
            mma_commit(&bar_m1);
        }
    } else if (warp == 17 && lane == 0) {
        // ---------------- TMA loads and stores
        int item = item0, k = k0, gg = gg0, bb = bb0;
        int row0 = bb * P.T + k * LT;
        uint32_t hc = 0, ic = 0;
        auto load_xy_at = [&](int hh, int r0, int xb) {
            mbar_expect_tx(&bar_xy[xb], 2 * PANEL);
            tma_load_2d(sXY + (2 * xb) * PANEL, &P.mX, &bar_xy[xb], hh * HP, r0);
            tma_load_2d(sXY + (2 * xb + 1) * PANEL, &P.mdY, &bar_xy[xb], hh * HP, r0);
        };
        auto load_xy = [&](int hl) { load_xy_at(gg * hpg + hl, row0, (hc + hl) & 1); };
        auto load_hq = [&](int hl) {
            const int hh = gg * hpg + hl;
            const int srow = (int)((((size_t)bb * P.nt + k) * P.h + hh) * DN);
            mbar_expect_tx(&bar_hq, 2 * PANEL);
            tma_load_2d(sH, &P.mH, &bar_hq, 0, srow);
            tma_load_2d(sQ, &P.mQ, &bar_hq, 0, srow);
        };
        auto load_item = [&]() {  // C and B of the item, H / Q of its first head
            mbar_expect_tx(&bar_cb, 4 * PANEL);
            tma_load_2d(sC, &P.mC, &bar_cb, gg * DN, row0);
            tma_load_2d(sC + PANEL, &P.mC, &bar_cb, gg * DN + 64, row0);
            tma_load_2d(sB, &P.mB, &bar_cb, gg * DN, row0);
            tma_load_2d(sB + PANEL, &P.mB, &bar_cb, gg * DN + 64, row0);
            load_hq(0);
        };
        prefetch_tmap(&P.mX);
        prefetch_tmap(&P.mdY);
        prefetch_tmap(&P.mH);
        prefetch_tmap(&P.mQ);
        load_xy(0);
        load_item();
        if (hpg > 1) load_xy(1);
        for (;;) {
            const int nitem = item + (int)gridDim.x;
            const bool more = nitem < P.items;
            const int nk = nitem % P.nt, ngg = (nitem / P.nt) % ngroups, nbb = nitem / (P.nt * ngroups);
            for (int hl = 0; hl < hpg; ++hl) {
                const uint32_t hcur = hc + hl;
                const int hh = gg * hpg + hl;
                const uint32_t ph = hcur & 1;
                // H, Q and this head's x / dy are free once the dC / dB products have completed (the last of the head to read
                // the panels) and every row has taken its dy values (they do before the arrive on bar_e)
                mbar_wait(&bar_m2b, ph, &failed);
                mbar_wait_spin(&bar_e, ph, &failed);
                if (hl + 1 < hpg) {
                    load_hq(hl + 1);
                    if (hl + 2 < hpg) load_xy(hl + 2);
                } else if (more) {
                    // x / dy of the next item's first head into the buffer of the head before this one (this head's
                    // buffer stages dB at the end of the item)
                    load_xy_at(ngg * hpg, nbb * P.T + nk * LT, (hcur + 1) & 1);
                }
                mbar_wait_spin(&bar_c, ph, &failed);    // dx staged
                tma_store_2d(&P.mdX, sdX, hh * HP, row0);
                tma_store_commit();
                tma_store_wait_read();
                mbar_arrive(&bar_sr);  // the dx staging panel may be rewritten
            }
            mbar_wait(&bar_m3, ic & 1, &failed);
            // C, B, H, Q are free now: the next item's loads go out before this item's group terms are stored
            const uint32_t hlast = hc + hpg - 1;
            const int st_gg = gg, st_row0 = row0;
            uint8_t* sdBst = sXY + (2 * (hlast & 1)) * PANEL;  // dB staging: the last head's x / dy buffer
            const uint32_t ic_done = ic;
            item = nitem;
            hc += hpg;
            ic += 1;
            if (more) {
                k = nk;
                gg = ngg;
                bb = nbb;
                row0 = bb * P.T + k * LT;
                load_item();
            }
            mbar_wait_spin(&bar_g2, ic_done & 1, &failed);  // dC and dB staged
            tma_store_2d(&P.mdC, sG, st_gg * DN, st_row0);
            tma_store_2d(&P.mdC, sG + PANEL, st_gg * DN + 64, st_row0);
            tma_store_2d(&P.mdB, sdBst, st_gg * DN, st_row0);
            tma_store_2d(&P.mdB, sdBst + PANEL, st_gg * DN + 64, st_row0);
            tma_store_commit();
            tma_store_wait_read();  // shared memory must outlive the reads only (the writes complete with the kernel)
            if (!more) break;
            mbar_arrive(&bar_sr2);
            if (hpg > 1) load_xy(1);
        }
    }
    __syncwarp();
  } else {
    // ======================= row warps: thread = (row, column quarter) =======================
    setmaxnreg_inc<kBwdRegsRow>();
    int item = item0, k = k0, gg = gg0, bb = bb0;
    uint32_t hc = 0, ic = 0;
    auto pos_of = [&](int hl) { return ((size_t)bb * P.h + gg * hpg + hl) * P.T + (size_t)k * LT; };
    const int rb = row >> 5;                   // row block, warp-uniform
    const bool active = qc <= rb, diag = qc == rb;
    const uint32_t lanes = lane_base(warp);
    // every lane fences its own writes, the warp converges, one lane arrives for all
    auto warp_arrive = [&](uint64_t* bar) {
        __syncwarp();
        mbar_arrive_if(bar, lane == 0);
    };
    // G panel and 16-byte chunk of this thread's two 16-column steps
    uint8_t* sGq = sG + (qc >> 1) * PANEL;
    const int gch = (qc & 1) * 4;

    for (;;) {
        float2 dS2[16];  // sum over heads of dS for this thread's 32 columns, as fp32 pairs
#pragma unroll
        for (int q = 0; q < 16; ++q) dS2[q] = make_float2(0.f, 0.f);
        // the item after this one (its row scalars are fetched during the last head of this one)
        const int nitem = item + (int)gridDim.x;
        const bool more = nitem < P.items;
        const int nk = nitem % P.nt, ngg = (nitem / P.nt) % ngroups, nbb = nitem / (P.nt * ngroups);

        for (int hl = 0; hl < hpg; ++hl) {
            const uint32_t hcur = hc + hl;
            const int hh = gg * hpg + hl, xb = hcur & 1, buf = hcur & 1;
            const uint32_t ph = hcur & 1;
            const size_t tpos = pos_of(hl) + row;
            if (qc == 0) {
                if (hl + 1 < hpg) fetch_scalars((hcur + 1) & 1, pos_of(hl + 1), hh + 1);
                else if (more) fetch_scalars((hcur + 1) & 1, ((size_t)nbb * P.h + ngg * hpg) * P.T + (size_t)nk * LT, ngg * hpg);
            }
            const float c_i = scum2[buf * LT + row], dtv = sdt[buf * LT + row], Dh = sD[buf * LT + row];
            mbar_wait(&bar_xy[xb], (hcur >> 1) & 1, &failed);
            uint8_t* sX = sXY + (2 * xb) * PANEL;
            uint8_t* sdY = sX + PANEL;
            const float Sk = scum2[buf * LT + LT - 1];
            // this thread's quarter row of x (raw); dy stays raw in shared memory and is re-read where needed
            uint32_t xr[8];
#pragma unroll
            for (int ch = 0; ch < 2; ++ch) {
                uint4 v = *reinterpret_cast<const uint4*>(sX + sw128(row, qc * 2 + ch));
                xr[ch * 4 + 0] = v.x; xr[ch * 4 + 1] = v.y; xr[ch * 4 + 2] = v.z; xr[ch * 4 + 3] = v.w;
            }
            float dyx = 0.f;  // sum_p dy[i,p] x[i,p] is the diagonal entry of dG = dY x^T: picked up in the mask loop
            const float ei = exp2f(c_i);
            const float dj = exp2f(Sk - c_i);
            mbar_wait(&bar_m1, ph, &failed);
            tc_fence_after();
            float2 rowacc2 = make_float2(0.f, 0.f);
            if (active) {
                const float rf = exp2f(c_i - scum2[buf * LT + qc * 32 + 31]);
                const float2 rf2 = make_float2(rf, rf);
#pragma unroll
                for (int sub = 0; sub < 2; ++sub) {
                    const int c0 = qc * 32 + sub * 16;
                    uint32_t rs[16], rg[16];
                    tmem_ld16(tS + lanes + c0, rs);
                    tmem_ld16(tdG + lanes + c0, rg);
                    const float2* F2 = reinterpret_cast<const float2*>(sfL + buf * LT + c0);
                    const float2* T2 = reinterpret_cast<const float2*>(sdt + buf * LT + c0);
                    tmem_ld_wait();
                    // Everything in fp32 pairs (one instruction, two columns).  rowacc uses the bf16-rounded G that
                    // the dX product reads (unpacked from the packed pair), so that the row and column sums of
                    // dG o G cancel exactly.
                    const float2* S2 = reinterpret_cast<const float2*>(rs);
                    const float2* G2 = reinterpret_cast<const float2*>(rg);
                    uint32_t gp[8];
                    const float2* C2 = reinterpret_cast<const float2*>(scum2 + buf * LT + c0);
#pragma unroll
                    for (int q2 = 0; q2 < 8; ++q2) {
                        float2 l;
                        if (EXACT && diag) {  // see the forward walk: the diagonal block entry by entry
                            const float2 cj = C2[q2];
                            l.x = exp2f(c_i - cj.x);
                            l.y = exp2f(c_i - cj.y);
                        } else {
                            l = mul2(rf2, F2[q2]);
                        }
                        if (diag) {  // columns beyond the row are masked
                            if (c0 + 2 * q2 > row) l.x = 0.f;
                            if (c0 + 2 * q2 + 1 > row) l.y = 0.f;
                        }
                        const float2 dg = mul2(G2[q2], T2[q2]);
                        const float2 gl = mul2(S2[q2], l);
                        const uint32_t pk = pack_bf16(gl.x, gl.y);
                        dS2[sub * 8 + q2] = fma2(dg, l, dS2[sub * 8 + q2]);
                        rowacc2 = fma2(dg, make_float2(__uint_as_float(pk << 16), __uint_as_float(pk & 0xffff0000u)), rowacc2);
                        gp[q2] = pk;
                    }
                    if (diag) {
#pragma unroll
                        for (int q = 0; q < 16; ++q)
                            if (c0 + q == row) dyx = __uint_as_float(rg[q]);
                    }
                    *reinterpret_cast<uint4*>(sGq + sw128(row, gch + sub * 2)) = make_uint4(gp[0], gp[1], gp[2], gp[3]);
                    *reinterpret_cast<uint4*>(sGq + sw128(row, gch + sub * 2 + 1)) = make_uint4(gp[4], gp[5], gp[6], gp[7]);
                }
            } else {
                if (hl == 0) {
                    // above the diagonal G is zero for every head: written once (the G panels are staging only after the loop)
                    const uint4 z = make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
                    for (int ch = 0; ch < 4; ++ch) *reinterpret_cast<uint4*>(sGq + sw128(row, gch + ch)) = z;
                }
            }
            const float rowacc = rowacc2.x + rowacc2.y;
            // (A) this thread's part of G is complete and its S / dG entries are read: the control warp issues dX1, dX2, Yo
            tc_fence_before();
            fence_async_smem();
            warp_arrive(&bar_a);
            // dYe goes where the last column quarter of dG was: the rows 96-127 wait for their quarter-3 warp to have read it
            if (rb == 3) named_bar_sync(2, 128);
            {   // Xd = d dt x in place (A operand of dB += Xd Q); dYe = e dY as bf16 pairs in TMEM
                uint32_t a[8];
                const __nv_bfloat162 wx2 = __float2bfloat162_rn(dj * dtv), we2 = __float2bfloat162_rn(ei);
#pragma unroll
                for (int ch = 0; ch < 2; ++ch) {
                    uint4 v, u = *reinterpret_cast<const uint4*>(sdY + sw128(row, qc * 2 + ch));
                    uint32_t* vv = reinterpret_cast<uint32_t*>(&v);
                    uint32_t* uu = reinterpret_cast<uint32_t*>(&u);
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        __nv_bfloat162 rx = __hmul2(*reinterpret_cast<__nv_bfloat162*>(&xr[ch * 4 + q]), wx2);
                        __nv_bfloat162 ry = __hmul2(*reinterpret_cast<__nv_bfloat162*>(&uu[q]), we2);
                        vv[q] = *reinterpret_cast<uint32_t*>(&rx);
                        a[ch * 4 + q] = *reinterpret_cast<uint32_t*>(&ry);
                    }
                    *reinterpret_cast<uint4*>(sX + sw128(row, qc * 2 + ch)) = v;
                }
                tmem_st8(tYe + lanes + qc * 8, a);
                tmem_st_wait();
            }
            // (B) Xd, dYe complete: the control warp issues dC, dB
            tc_fence_before();
            fence_async_smem();
            warp_arrive(&bar_b);
            // While the products run: <Q, H> of the head.  Both panels are [n][p] bf16 in the same layout, so the products
            // pair up chunk by chunk whatever the swizzle; 1024 chunks of 16 bytes, two per thread.
            float qh_acc;
            {
                mbar_wait(&bar_hq, ph, &failed);  // long complete; every reader of the panels observes the barrier itself
                float2 q2 = make_float2(0.f, 0.f);
#pragma unroll
                for (int i = 0; i < 2; ++i) {
                    const int c = tid + 512 * i;
                    const uint4 hv = *reinterpret_cast<const uint4*>(sH + c * 16);
                    const uint4 qv = *reinterpret_cast<const uint4*>(sQ + c * 16);
                    const uint32_t* hu = reinterpret_cast<const uint32_t*>(&hv);
                    const uint32_t* qu = reinterpret_cast<const uint32_t*>(&qv);
#pragma unroll
                    for (int q = 0; q < 4; ++q)
                        q2 = fma2(__bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&hu[q])),
                                  __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&qu[q])), q2);
                }
                qh_acc = q2.x + q2.y;
            }
            float ddt_acc, st_acc, yo_acc;
            {
                uint32_t yr[8];
#pragma unroll
                for (int ch = 0; ch < 2; ++ch) {
                    uint4 u = *reinterpret_cast<const uint4*>(sdY + sw128(row, qc * 2 + ch));
                    yr[ch * 4 + 0] = u.x; yr[ch * 4 + 1] = u.y; yr[ch * 4 + 2] = u.z; yr[ch * 4 + 3] = u.w;
                }
                // e_i <dY_i, Yo_i> over this thread's 16 columns (Yo = C H^T is the first product of the group)
                mbar_wait(&bar_m2y, ph, &failed);
                tc_fence_after();
                {
                    uint32_t o[16];
                    tmem_ld16(tYo + lanes + qc * 16, o);
                    tmem_ld_wait();
                    float2 r2 = make_float2(0.f, 0.f);
                    const float2* O2 = reinterpret_cast<const float2*>(o);
#pragma unroll
                    for (int q = 0; q < 8; ++q)
                        r2 = fma2(O2[q], __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&yr[q])), r2);
                    yo_acc = ei * (r2.x + r2.y);
                }
                mbar_wait(&bar_m2, ph, &failed);
                tc_fence_after();
                // fp32 pairs throughout: e = dX1 + d dX2, dx = dt e + D dy, and the two row sums <e, x>, <dX2, x>
                float2 ddt2 = make_float2(0.f, 0.f), st2 = make_float2(0.f, 0.f);
                const float2 dt2 = make_float2(dtv, dtv), D2 = make_float2(Dh, Dh);
                uint32_t a[16], b2[16];
                tmem_ld16(tX1 + lanes + qc * 16, a);
                tmem_ld16(tX2 + lanes + qc * 16, b2);
                tmem_ld_wait();
                // (E) Yo, dX1 and dX2 are in registers: the accumulators of this head may be overwritten.  The weight d_j that
                // every product below starts from is chosen, by a bit of the arrive's token, between two copies of the same
                // number (the second from a fresh read of the row's log-decay), which ties the arithmetic to the arrive.
                tc_fence_before();
                __syncwarp();
                const uint32_t tok = mbar_arrive_if_token(&bar_e, lane == 0);
                const float dj_b = exp2f(Sk - *reinterpret_cast<volatile float*>(&scum2[buf * LT + row]));
                const float dj_e = (tok & 1u) ? dj_b : dj;
                const float2 dj2 = make_float2(dj_e, dj_e);
                const float2* A2 = reinterpret_cast<const float2*>(a);
                const float2* S2 = reinterpret_cast<const float2*>(b2);
                uint32_t dxp[8];
#pragma unroll
                for (int q = 0; q < 8; ++q) {
                    const float2 fx = __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&xr[q]));
                    const float2 fy = __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&yr[q]));
                    const float2 e = fma2(dj2, S2[q], A2[q]);
                    ddt2 = fma2(e, fx, ddt2);
                    st2 = fma2(S2[q], fx, st2);
                    const float2 o = fma2(D2, fy, mul2(e, dt2));
                    dxp[q] = pack_bf16(o.x, o.y);
                }
                *reinterpret_cast<uint4*>(sdX + sw128(row, qc * 2)) = make_uint4(dxp[0], dxp[1], dxp[2], dxp[3]);
                *reinterpret_cast<uint4*>(sdX + sw128(row, qc * 2 + 1)) = make_uint4(dxp[4], dxp[5], dxp[6], dxp[7]);
                ddt_acc = ddt2.x + ddt2.y;
                st_acc = st2.x + st2.y;
            }
            // (C) dx staged: the TMA lane stores it
            tc_fence_before();
            fence_async_smem();
            warp_arrive(&bar_c);
            {
                // gradient w.r.t. the tile-cumulative log-decay of this row, one partial per quarter, summed after the
                // barrier; the terms that act through S = cum[127] (state weights d_j, and the decay of the entering
                // state) are summed per warp
                sred[(0 * 4 + qc) * LT + row] = (rowacc - dtv * ddt_acc) + yo_acc;
                sred[(1 * 4 + qc) * LT + row] = ddt_acc;
                sred[(2 * 4 + qc) * LT + row] = dyx;
                float red = dj * dtv * st_acc + exp2f(Sk) * qh_acc;
#pragma unroll
                for (int of = 16; of > 0; of >>= 1) red += __shfl_xor_sync(0xffffffffu, red, of);
                if (lane == 0) swred[warp] = red;
            }
            if (qc == 0 && hl + 1 < hpg) finish_scalars((hcur + 1) & 1);
            named_bar_sync(1, 512);  // partial sums and the next head's column arrays visible to the row warps
            if (qc == 0) {
                // fixed order: deterministic
                P.g[tpos] = (sred[0 * LT + row] + sred[1 * LT + row]) + (sred[2 * LT + row] + sred[3 * LT + row]);
                P.ddtx[tpos] = (sred[4 * LT + row] + sred[5 * LT + row]) + (sred[6 * LT + row] + sred[7 * LT + row]);
                P.dyx[tpos] = (sred[8 * LT + row] + sred[9 * LT + row]) + (sred[10 * LT + row] + sred[11 * LT + row]);
                if (row < 8) P.gS[((((size_t)bb * P.h + hh) * P.nt) + k) * 8 + row] = swred[row] + swred[row + 8];
            }
        }
        // ---- group terms: stage sum_h dS as bf16 [i][j] (panel = column half) in the H / Q panels for the two
        // closing products
        const uint32_t hlast = hc + hpg - 1;
        mbar_wait(&bar_m2b, hlast & 1, &failed);  // the last head's products have read H, Q, Xd / dY
        {
            float v[32];
#pragma unroll
            for (int q = 0; q < 16; ++q) {
                v[2 * q] = dS2[q].x;
                v[2 * q + 1] = dS2[q].y;
            }
            store_half_row(sH + (qc >> 1) * PANEL, row, gch, v);
        }
        tc_fence_before();
        fence_async_smem();
        warp_arrive(&bar_g1);
        mbar_wait(&bar_m3, ic & 1, &failed);
        tc_fence_after();
        uint8_t* sdBst = sXY + (2 * (hlast & 1)) * PANEL;  // dB staging: the last head's x / dy buffer
        item = nitem;
        hc += hpg;
        ic += 1;
        if (more) {
            k = nk;
            gg = ngg;
            bb = nbb;
        }
        {
            uint32_t a[32], b2[32];
            tmem_ld32(tdC + lanes + qc * 32, a);
            tmem_ld32(tdB + lanes + qc * 32, b2);
            tmem_ld_wait();
            float va[32];
#pragma unroll
            for (int q = 0; q < 32; ++q) va[q] = __uint_as_float(a[q]);
            store_half_row(sG + (qc >> 1) * PANEL, row, gch, va);
#pragma unroll
            for (int q = 0; q < 32; ++q) va[q] = __uint_as_float(b2[q]);
            store_half_row(sdBst + (qc >> 1) * PANEL, row, gch, va);
        }
        if (qc == 0 && more) finish_scalars(hc & 1);
        tc_fence_before();
        fence_async_smem();
        warp_arrive(&bar_g2);  // dC, dB staged and read out of TMEM: the control warp stores them
        named_bar_sync(1, 512);  // the first head's column arrays visible to the row warps
        if (!more) break;
    }
  }
    tc_fence_before();
    __syncthreads();
    if (tid == 0 && failed) atomicExch(P.status, 1);
    if (warp == 1) tmem_dealloc(tm, 512);
}

}  // namespace tc
}  // namespace ssd
