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
// 512 threads: thread = (row, column quarter).  TMEM lanes are tied to warp % 4, so the rows 96-127, whose
// causal rows are the longest, can only be read by the warps of one SM sub-partition; four warps per 32-row
// block walk two 16-column steps each per head, and a quarter is exactly one 32-column block of the causal
// mask (active iff quarter <= row block, diagonal iff equal).  Row 0 of the last quarter, whose mask work is
// all zeros, also issues every TMA copy and tcgen05.mma.  Per head:
//   S, dG -> mask loop (G -> smem, dS summed over heads in registers) -> [barrier A] -> dX1, dX2 issued;
//   meanwhile Xd = d dt x in place and dYe = e dY -> TMEM -> [mbarrier B, control only] -> dC, dB products
//   issued -> row epilogue on dX1, dX2 -> [barrier C] -> S, dG of the next head issued, dx stored.
// x / dy tiles are double-buffered across heads; H / Q are reloaded as soon as the dC / dB products complete.
// The per-row sums (gradient of the tile-cumulative log-decay, <dX, x>, <dy, x>) are summed over the four
// quarters in shared memory and leave the kernel as one array each.
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


// 13 operand panels | scum2, sfL, sdt [2][128] | row partials [3][4][128] | warp partials [16] | alignment slack
constexpr size_t kBwdSmem = 13 * PANEL + 6 * LT * 4 + 12 * LT * 4 + 64 + 1024;

// Two instantiations (EXACT: diagonal mask blocks entry by entry, see kMaskSafeLog2); both are launched and the
// extreme-decay flag decides on the device which of the two does the work (kept as separate kernels: as an
// out-of-line body this kernel loses registers to the call and spills).
template <bool EXACT>
__global__ void __launch_bounds__(512, 1) bwd_tile_kernel(const __grid_constant__ BwdParams P) {
    if ((P.extreme[0] != 0) != EXACT) return;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* sm = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    uint8_t* sC = sm;                  // 2 panels [pos][n]
    uint8_t* sB = sC + 2 * PANEL;      // 2 panels [pos][n]
    uint8_t* sG = sB + 2 * PANEL;      // 2 panels [i][j]; at the end dC staging
    uint8_t* sXY = sG + 2 * PANEL;     // 4 panels: x0, dy0, x1, dy1; at the end sum_h dS (2) and dB staging (2)
    uint8_t* sH = sXY + 4 * PANEL;     // [n][p]
    uint8_t* sQ = sH + PANEL;          // [n][p]
    uint8_t* sdX = sQ + PANEL;         // dx staging
    float* scum2 = reinterpret_cast<float*>(sdX + PANEL);  // [2][128] each:
    float* sfL = scum2 + 2 * LT;       //   2^(cend - c_j)
    float* sdt = sfL + 2 * LT;         //   dt_j
    float* sred = sdt + 2 * LT;        // [3][4][128]: per-quarter partials of g, ddtx, dyx of the current head
    float* swred = sred + 12 * LT;     // [16]: per-warp partials of the S-borne term
    __shared__ uint64_t bar_cb, bar_xy[2], bar_hq, bar_m1, bar_m2, bar_m2b, bar_m3, bar_b;
    __shared__ uint32_t tmem_slot;
    __shared__ int failed;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    // Persistent over work items (tile k, group gg, batch bb): the loads and the per-row scalars of the next item
    // are issued while the group terms of the current one are stored.  `hc` counts heads and `ic` items since the
    // start of the kernel; every buffer index and mbarrier phase derives from them.
    const int hpg = P.hpg, ngroups = P.h / P.hpg;
    int item = blockIdx.x;
    int k = item % P.nt, gg = (item / P.nt) % ngroups, bb = item / (P.nt * ngroups);
    int row0 = bb * P.T + k * LT;
    uint32_t hc = 0, ic = 0;
    const int row = tid & 127, qc = tid >> 7;  // column quarter: S / dG columns [32 qc, 32 qc + 32), p columns [16 qc, +16)
    const int rb = row >> 5;                   // row block, warp-uniform
    const bool active = qc <= rb, diag = qc == rb;
    // control thread: row 0 of the last quarter, whose mask work is all zeros
    constexpr int CTL = 384;

    if (tid == 0) {
        failed = 0;
        mbar_init(&bar_cb, 1);
        mbar_init(&bar_xy[0], 1);
        mbar_init(&bar_xy[1], 1);
        mbar_init(&bar_hq, 1);
        mbar_init(&bar_m1, 1);
        mbar_init(&bar_m2, 1);
        mbar_init(&bar_m2b, 1);
        mbar_init(&bar_m3, 1);
        mbar_init(&bar_b, 512);
        mbar_fence_init();
    }
    if (warp == 1) {
        tmem_alloc(&tmem_slot, 512);
        tmem_relinquish();
    }
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
    auto pos_of = [&](int hl) { return ((size_t)bb * P.h + gg * hpg + hl) * P.T + (size_t)k * LT; };
    // per-head row scalars are fetched one head ahead; the shared per-column arrays of head hl + 1 are
    // written before the last block-wide barrier of head hl
    float c_n = P.tcum[pos_of(0) + row], cend_n = P.tcum[pos_of(0) + (row | 31)];
    float dt_n = P.dtT ? P.dtT[pos_of(0) + row] : 1.f;
    float D_n = P.skipT ? P.skipT[pos_of(0) + row] : (P.D ? P.D[gg * hpg] : 0.f);
    auto publish_columns = [&](int buf) {
        if (qc == 0) {
            scum2[buf * LT + row] = c_n;
            sfL[buf * LT + row] = exp2f(cend_n - c_n);
            sdt[buf * LT + row] = dt_n;
        }
    };
    publish_columns(0);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    auto load_item = [&]() {  // C and B of the item, H / Q of its first head
        mbar_expect_tx(&bar_cb, 4 * PANEL);
        tma_load_2d(sC, &P.mC, &bar_cb, gg * DN, row0);
        tma_load_2d(sC + PANEL, &P.mC, &bar_cb, gg * DN + 64, row0);
        tma_load_2d(sB, &P.mB, &bar_cb, gg * DN, row0);
        tma_load_2d(sB + PANEL, &P.mB, &bar_cb, gg * DN + 64, row0);
        load_hq(0);
    };
    if (tid == CTL) {
        load_xy(0);
        load_item();
    }
    const uint32_t tm = tmem_slot;
    // phase 1: S [0,128) dG [128,256); after the mask loop (barrier A) dX1 [0,64) and dX2 [64,128) take the S
    // columns, dYe (bf16 pairs) the dG columns [128,160) and Yo = C H^T the dG columns [160,224); persistent over
    // heads: dC [256,384) dB [384,512)
    const uint32_t tS = tm, tdG = tm + 128, tX1 = tm, tX2 = tm + 64, tYo = tm + 160, tdC = tm + 256, tdB = tm + 384;
    const uint32_t lanes = lane_base(warp);
    const uint32_t c0a = smem_u32(sC), b0a = smem_u32(sB), g0a = smem_u32(sG), h0a = smem_u32(sH), q0a = smem_u32(sQ);
    auto issue_phase1 = [&](int hl, bool commit) {  // S = C B^T (K = n) and dG = dY x^T (K = p) of head hl
        const uint32_t x0 = smem_u32(sXY + (2 * ((hc + hl) & 1)) * PANEL), y0 = x0 + PANEL;
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
            const uint32_t off = (kk >> 2) * PANEL + (kk & 3) * 32;
            mma_ss(tS, smem_desc(c0a + off, 16, 1024), smem_desc(b0a + off, 16, 1024), kIdescKK128, kk > 0);
        }
#pragma unroll
        for (int kk = 0; kk < 4; ++kk)
            mma_ss(tdG, smem_desc(y0 + kk * 32, 16, 1024), smem_desc(x0 + kk * 32, 16, 1024), kIdescKK128, kk > 0);
        if (commit) mma_commit(&bar_m1);
    };

    // G panel and 16-byte chunk of this thread's two 16-column steps
    uint8_t* sGq = sG + (qc >> 1) * PANEL;
    const int gch = (qc & 1) * 4;

  for (;;) {
    float2 dS2[16];  // sum over heads of dS for this thread's 32 columns, as fp32 pairs
#pragma unroll
    for (int q = 0; q < 16; ++q) dS2[q] = make_float2(0.f, 0.f);
    mbar_wait(&bar_cb, ic & 1, &failed);
    if (tid == CTL && ic == 0) {  // later items: issued at the end of the item before
        mbar_wait(&bar_xy[hc & 1], (hc >> 1) & 1, &failed);
        tc_fence_after();
        issue_phase1(0, true);
        if (hpg > 1) load_xy(1);
    }
    // the item after this one (its row scalars are fetched during the last head of this one)
    const int nitem = item + (int)gridDim.x;
    const bool more = nitem < P.items;
    const int nk = nitem % P.nt, ngg = (nitem / P.nt) % ngroups, nbb = nitem / (P.nt * ngroups);

    for (int hl = 0; hl < hpg; ++hl) {
        const uint32_t hcur = hc + hl;
        const int hh = gg * hpg + hl, xb = hcur & 1, buf = hcur & 1;
        const uint32_t ph = hcur & 1;
        const size_t tpos = pos_of(hl) + row;
        const float c_i = c_n, dtv = dt_n, Dh = D_n;
        if (hl + 1 < hpg) {
            const size_t o = pos_of(hl + 1);
            c_n = P.tcum[o + row];
            cend_n = P.tcum[o + (row | 31)];
            dt_n = P.dtT ? P.dtT[o + row] : 1.f;
            D_n = P.skipT ? P.skipT[o + row] : (P.D ? P.D[hh + 1] : 0.f);
        } else if (more) {
            const size_t o = ((size_t)nbb * P.h + ngg * hpg) * P.T + (size_t)nk * LT;
            c_n = P.tcum[o + row];
            cend_n = P.tcum[o + (row | 31)];
            dt_n = P.dtT ? P.dtT[o + row] : 1.f;
            D_n = P.skipT ? P.skipT[o + row] : (P.D ? P.D[ngg * hpg] : 0.f);
        }
        mbar_wait(&bar_xy[xb], (hcur >> 1) & 1, &failed);
        uint8_t* sX = sXY + (2 * xb) * PANEL;
        uint8_t* sdY = sX + PANEL;
        const uint32_t x0 = smem_u32(sX), y0 = x0 + PANEL;  // phase 1 of this head was issued one step earlier
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
        } else if (hl == 0) {
            // above the diagonal G is zero for every head: written once (the G panels are staging only after the loop)
            const uint4 z = make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
            for (int ch = 0; ch < 4; ++ch) *reinterpret_cast<uint4*>(sGq + sw128(row, gch + ch)) = z;
        }
        const float rowacc = rowacc2.x + rowacc2.y;
        if (tid == CTL) tma_store_wait_read();  // the previous head's dx store has read sdX
        tc_fence_before();
        fence_async_smem();
        __syncthreads();  // (A) G complete, S and dG read by everyone
        if (tid == CTL) {
            mbar_wait(&bar_hq, ph, &failed);  // H and Q of this head have landed
            tc_fence_after();
#pragma unroll
            for (int kk = 0; kk < 8; ++kk)  // dX1 = G^T dY : A = G MN-major (M = j, K = i), B = dY MN-major
                mma_ss(tX1, smem_desc(g0a + kk * 2048, PANEL, 1024), smem_desc(y0 + kk * 2048, PANEL, 1024), kIdescMM, kk > 0);
#pragma unroll
            for (int kk = 0; kk < 8; ++kk) {  // dX2 = B Q^T : A = B K-major (K = n), B = Q^T [n][p] MN-major
                const uint32_t off = (kk >> 2) * PANEL + (kk & 3) * 32;
                mma_ss(tX2, smem_desc(b0a + off, 16, 1024), smem_desc(q0a + kk * 2048, PANEL, 1024), kIdescKM, kk > 0);
            }
#pragma unroll
            for (int kk = 0; kk < 8; ++kk) {  // Yo = C H^T : A = C K-major (K = n), B = H^T [n][p] MN-major
                const uint32_t off = (kk >> 2) * PANEL + (kk & 3) * 32;
                mma_ss(tYo, smem_desc(c0a + off, 16, 1024), smem_desc(h0a + kk * 2048, PANEL, 1024), kIdescKM, kk > 0);
            }
            mma_commit(&bar_m2);  // the row epilogue needs dX1, dX2 and Yo
        }
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
            tmem_st8(tdG + lanes + qc * 8, a);
            tmem_st_wait();
        }
        // (B) Xd, dYe complete: only the control thread waits for it, the others go on to the row epilogue
        tc_fence_before();
        fence_async_smem();
        mbar_arrive(&bar_b);
        if (tid == CTL) {
            mbar_wait(&bar_b, ph, &failed);
            tc_fence_after();
#pragma unroll
            for (int kk = 0; kk < 4; ++kk)  // dC += dYe H : A in TMEM (K = p), B = H^T [n][p] K-major, N = 128
                mma_ts(tdC, tdG + kk * 8, smem_desc(h0a + kk * 32, 16, 1024), kIdescKK128, hl > 0 || kk > 0);
#pragma unroll
            for (int kk = 0; kk < 4; ++kk)  // dB += Xd Q : A = Xd K-major (in place of x), B = Q^T [n][p] K-major
                mma_ss(tdB, smem_desc(x0 + kk * 32, 16, 1024), smem_desc(q0a + kk * 32, 16, 1024), kIdescKK128, hl > 0 || kk > 0);
            mma_commit(&bar_m2b);  // releases H, Q, Xd and the dYe columns
        }
        mbar_wait(&bar_m2, ph, &failed);
        tc_fence_after();
        float ddt_acc, st_acc, qh_acc, yo_acc;
        {
            // fp32 pairs throughout: e = dX1 + d dX2, dx = dt e + D dy, and the two row sums <e, x>, <dX2, x>
            float2 ddt2 = make_float2(0.f, 0.f), st2 = make_float2(0.f, 0.f);
            const float2 dj2 = make_float2(dj, dj), dt2 = make_float2(dtv, dtv), D2 = make_float2(Dh, Dh);
            uint32_t a[16], b2[16], yr[8];
            tmem_ld16(tX1 + lanes + qc * 16, a);
            tmem_ld16(tX2 + lanes + qc * 16, b2);
#pragma unroll
            for (int ch = 0; ch < 2; ++ch) {
                uint4 u = *reinterpret_cast<const uint4*>(sdY + sw128(row, qc * 2 + ch));
                yr[ch * 4 + 0] = u.x; yr[ch * 4 + 1] = u.y; yr[ch * 4 + 2] = u.z; yr[ch * 4 + 3] = u.w;
            }
            tmem_ld_wait();
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
            // <Q, H> over this thread's 16 columns of state row n = `row` (both panels are [n][p] bf16; they stay put
            // until the products that read them have completed, which is after the closing barrier of the head)
            {
                mbar_wait(&bar_hq, ph, &failed);  // long complete; every reader of the panels observes the barrier itself
                float2 q2 = make_float2(0.f, 0.f);
#pragma unroll
                for (int ch = 0; ch < 2; ++ch) {
                    const uint4 hv = *reinterpret_cast<const uint4*>(sH + sw128(row, qc * 2 + ch));
                    const uint4 qv = *reinterpret_cast<const uint4*>(sQ + sw128(row, qc * 2 + ch));
                    const uint32_t* hu = reinterpret_cast<const uint32_t*>(&hv);
                    const uint32_t* qu = reinterpret_cast<const uint32_t*>(&qv);
#pragma unroll
                    for (int q = 0; q < 4; ++q)
                        q2 = fma2(__bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&hu[q])),
                                  __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&qu[q])), q2);
                }
                qh_acc = q2.x + q2.y;
            }
            // e_i <dY_i, Yo_i> over this thread's 16 columns (Yo = C H^T came with dX1 and dX2)
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
        }
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
        if (hl + 1 < hpg) publish_columns((hcur + 1) & 1);
        tc_fence_before();
        fence_async_smem();
        __syncthreads();  // (C) dx staged, TMEM reads done, partial sums and next head's column arrays visible
        if (qc == 0) {
            // fixed order: deterministic
            P.g[tpos] = (sred[0 * LT + row] + sred[1 * LT + row]) + (sred[2 * LT + row] + sred[3 * LT + row]);
            P.ddtx[tpos] = (sred[4 * LT + row] + sred[5 * LT + row]) + (sred[6 * LT + row] + sred[7 * LT + row]);
            P.dyx[tpos] = (sred[8 * LT + row] + sred[9 * LT + row]) + (sred[10 * LT + row] + sred[11 * LT + row]);
            if (row < 8) P.gS[((((size_t)bb * P.h + hh) * P.nt) + k) * 8 + row] = swred[row] + swred[row + 8];
        }
        if (tid == CTL) {
            // the products of the next head first (every thread waits for them), the stores and loads after
            mbar_wait(&bar_m2b, ph, &failed);  // dC / dB products of this head done: dYe, H, Q, Xd are free
            if (hl + 1 < hpg) {
                // everyone has read dX1 / dX2, so S and dG of the next head may overwrite them now; its x / dy
                // tiles were prefetched during this head
                mbar_wait(&bar_xy[xb ^ 1], ((hcur + 1) >> 1) & 1, &failed);
                tc_fence_after();
                issue_phase1(hl + 1, true);
            }
            tma_store_2d(&P.mdX, sdX, hh * HP, row0);
            tma_store_commit();
            if (hl + 1 < hpg) {
                load_hq(hl + 1);
                if (hl + 2 < hpg) load_xy(hl + 2);  // this head's x / dy buffer is free
            } else if (more) {
                // x / dy of the next item's first head into the buffer of the head before this one (this head's
                // buffer stages dB at the end of the item)
                load_xy_at(ngg * hpg, nbb * P.T + nk * LT, (hcur + 1) & 1);
            }
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
    __syncthreads();
    if (tid == CTL) {
        tc_fence_after();
        const uint32_t s0 = h0a;
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {  // dC += dS B : A = dS K-major (K = j), B = B [j][n] MN-major, N = 128
            const uint32_t off = (kk >> 2) * PANEL + (kk & 3) * 32;
            mma_ss(tdC, smem_desc(s0 + off, 16, 1024), smem_desc(b0a + kk * 2048, PANEL, 1024), kIdescKM128, true);
        }
#pragma unroll
        for (int kk = 0; kk < 8; ++kk)  // dB += dS^T C : A = dS MN-major (M = j, K = i), B = C [i][n] MN-major
            mma_ss(tdB, smem_desc(s0 + kk * 2048, PANEL, 1024), smem_desc(c0a + kk * 2048, PANEL, 1024), kIdescMM128, true);
        mma_commit(&bar_m3);
    }
    mbar_wait(&bar_m3, ic & 1, &failed);
    tc_fence_after();
    // C, B, H, Q and the x / dy buffer of the head before the last are free now: the next item's loads and row
    // scalars go out before this item's group terms are stored
    const int st_gg = gg, st_row0 = row0;
    uint8_t* sdBst = sXY + (2 * (hlast & 1)) * PANEL;  // dB staging: the last head's x / dy buffer
    item = nitem;
    hc += hpg;
    ic += 1;
    if (more) {
        k = nk;
        gg = ngg;
        bb = nbb;
        row0 = bb * P.T + k * LT;
        if (tid == CTL) load_item();
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
    if (more) publish_columns(hc & 1);
    tc_fence_before();
    fence_async_smem();
    __syncthreads();
    if (tid == CTL) {
        tma_store_2d(&P.mdC, sG, st_gg * DN, st_row0);
        tma_store_2d(&P.mdC, sG + PANEL, st_gg * DN + 64, st_row0);
        tma_store_2d(&P.mdB, sdBst, st_gg * DN, st_row0);
        tma_store_2d(&P.mdB, sdBst + PANEL, st_gg * DN + 64, st_row0);
        tma_store_commit();
        if (more) {  // S and dG of the next item's first head run while the stores read their staging panels
            mbar_wait(&bar_cb, ic & 1, &failed);
            mbar_wait(&bar_xy[hc & 1], (hc >> 1) & 1, &failed);
            tc_fence_after();
            issue_phase1(0, false);
        }
        // shared memory must outlive the reads only (the writes complete with the kernel); S and dG of the next
        // item are announced after this wait, and nobody overwrites the staging panels before that
        tma_store_wait_read();
        if (more) {
            mma_commit(&bar_m1);
            if (hpg > 1) load_xy(1);
        }
    }
    if (!more) break;
  }
    if (tid == CTL && failed) atomicExch(P.status, 1);
    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tm, 512);
}

}  // namespace tc
}  // namespace ssd
