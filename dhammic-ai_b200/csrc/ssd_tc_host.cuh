// Host side of the tensor-core path: tensor maps, workspace layout and launches.
#pragma once
#include <atomic>
#include <cstdio>

#include "../../include/ssd_b200.h"
#include "ssd_tc.cuh"

namespace ssd {
namespace tc {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// The driver entry point is looked up at run time so that the library links against the CUDA
// runtime only and loads on machines without a driver.
inline EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess) p = nullptr;
        return (EncodeTiledFn)p;
    }();
    return fn;
}

// 2D bf16 tensor [rows][cols] (cols contiguous), box 64 columns x 128 rows, 128-byte swizzle.
inline bool make_map(CUtensorMap* m, const void* base, uint64_t rows, uint64_t cols) {
    EncodeTiledFn enc = encode_fn();
    if (!enc) return false;
    cuuint64_t dims[2] = {cols, rows};
    cuuint64_t strides[1] = {cols * 2};
    cuuint32_t box[2] = {64, 128};
    cuuint32_t es[2] = {1, 1};
    return enc(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, es,
               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

struct Ws {
    size_t status, tcum, dtT, skipT, Hst, Qst, final_state, dinit, g, ddtx, dyx, gS, dAh_part, dD_part, total;
};

inline Ws ws_layout(const Dims& d, int pass) {
    Ws w{};
    size_t off = 0;
    auto take = [&](size_t bytes) {
        size_t o = off;
        off += (bytes + 255) / 256 * 256;
        return o;
    };
    const size_t bht = (size_t)d.b * d.h * d.T * 4;
    const size_t bhpn = (size_t)d.b * d.h * d.p * d.n * 4;
    const size_t st = (size_t)d.b * (d.T / LT) * d.h * DN * HP * 2;
    w.status = take(256);
    w.tcum = take(bht);
    w.dtT = take(bht);
    w.skipT = take(bht);
    if (pass == SSD_B200_PASS_BWD) {
        w.Hst = take(st);
        w.Qst = take(st);
        w.final_state = take(bhpn);
        w.dinit = take(bhpn);
        w.g = take(bht);
        w.ddtx = take(bht);
        w.dyx = take(bht);
        w.gS = take((size_t)d.b * d.h * (d.T / LT) * 8 * 4);
        w.dAh_part = take((size_t)d.b * (d.T / LT) * d.h * 4);
        w.dD_part = take((size_t)d.b * (d.T / LT) * d.h * 4);
    }
    w.total = off;
    return w;
}

inline size_t workspace_bytes(const Dims& d, int pass) { return ws_layout(d, pass).total; }
// The `states` buffer a forward call may fill for the backward call of the same inputs: the bf16 state entering
// every tile, followed by the three (b,h,T) fp32 arrays the tile kernels read (tile-cumulative log2 decay, dt and
// the per-position skip coefficient in (b,h,T) order) and the extreme-decay flag of tile_cumsum_kernel, so that the backward neither walks the states
// nor rebuilds those arrays.
inline size_t tile_states_bytes(const Dims& d) { return (size_t)d.b * (d.T / LT) * d.h * DN * HP * 2; }
inline size_t states_bytes(const Dims& d) { return tile_states_bytes(d) + 3 * ((size_t)d.b * d.h * d.T * 4) + 256; }

#define SSD_TC_FAIL(code, ...)              \
    do {                                    \
        snprintf(err, errn, __VA_ARGS__);   \
        return code;                        \
    } while (0)

#define SSD_TC_CHECK(what)                                                                        \
    do {                                                                                          \
        cudaError_t e_ = cudaGetLastError();                                                      \
        if (e_ != cudaSuccess) SSD_TC_FAIL(SSD_B200_ECUDA, "%s: %s", what, cudaGetErrorString(e_)); \
    } while (0)

inline int sm_count() {  // SMs of the current device (one persistent CTA each)
    int dev = 0, n = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)
        return 148;
    return n;
}

// Opt-in shared-memory sizes of the tensor-core kernels: set once per device and process (a function attribute
// lives as long as the device's context; after cudaDeviceReset a launch fails with an error code, it does not misbehave).
inline int set_walk_attrs(char* err, size_t errn) {
    static std::atomic<unsigned long long> done{0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) dev = 0;
    const unsigned long long bit = 1ull << (dev & 63);
    if (done.load(std::memory_order_acquire) & bit) return 0;
    const auto attr = cudaFuncAttributeMaxDynamicSharedMemorySize;
    cudaError_t e = cudaFuncSetAttribute(fwd_walk_kernel<false>, attr, (int)kFwdSmem);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(fwd_walk_kernel<true>, attr, (int)kFwdSmem);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(states_walk_kernel, attr, (int)WalkCfg<1>::SMEM);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(rev_walk_kernel<1>, attr, (int)RevCfg<1>::SMEM);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(rev_walk_kernel<2>, attr, (int)RevCfg<2>::SMEM);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(summary_kernel<false, 1>, attr, (int)SumCfg<1>::SMEM);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(summary_kernel<true, 1>, attr, (int)SumCfg<1>::SMEM);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(summary_kernel<false, 2>, attr, (int)SumCfg<2>::SMEM);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(summary_kernel<true, 2>, attr, (int)SumCfg<2>::SMEM);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(bwd_tile_kernel<false>, attr, (int)kBwdSmem);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(bwd_tile_kernel<true>, attr, (int)kBwdSmem);
    if (e != cudaSuccess) SSD_TC_FAIL(SSD_B200_ECUDA, "set shared memory size: %s", cudaGetErrorString(e));
    done.fetch_or(bit, std::memory_order_release);
    return 0;
}

inline int launch_tile_cumsum(const Dims& d, const float* cum, const float* dt, float* tcum, float* dtT, const float* skip,
                              float* skipT, int* extreme, cudaStream_t st, char* err, size_t errn) {
    dim3 g(d.T / LT, (d.h + 31) / 32, d.b);
    SSD_LAUNCH(prof::K_TC_AUX, st, tile_cumsum_kernel<<<g, 256, 0, st>>>(cum, dt, tcum, dtT, skip, skipT, extreme, d.b, d.T, d.h, d.l));
    SSD_TC_CHECK("tile_cumsum");
    return 0;
}

inline int forward(const ssd_b200_fwd_args* a, const Dims& d, cudaStream_t st, char* err, size_t errn) {
    Ws w = ws_layout(d, SSD_B200_PASS_FWD);
    if (a->workspace_bytes < w.total) SSD_TC_FAIL(SSD_B200_EWORKSPACE, "workspace %zu < %zu", a->workspace_bytes, w.total);
    if (!encode_fn()) SSD_TC_FAIL(SSD_B200_ECUDA, "cuTensorMapEncodeTiled is not available");
    const bool states_only = (a->flags & SSD_B200_FWD_STATES_ONLY) != 0;
    for (const void* p : {a->x, a->B, a->C, (const void*)a->y})
        if ((uintptr_t)p & 15) SSD_TC_FAIL(SSD_B200_EINVAL, "tensor-core path needs 16-byte aligned tensors");
    char* ws = (char*)a->workspace;
    int* status = (int*)(ws + w.status);
    float* tcum = (float*)(ws + w.tcum);
    float* dtT = a->dt ? (float*)(ws + w.dtT) : nullptr;
    float* skipT = a->skip ? (float*)(ws + w.skipT) : nullptr;
    int* extreme = status + 1;  // raised by tile_cumsum_kernel (see kMaskSafeLog2)
    const bool aux_valid = (a->flags & SSD_B200_FWD_AUX_VALID) != 0;
    if (aux_valid && !a->states) SSD_TC_FAIL(SSD_B200_EINVAL, "SSD_B200_FWD_AUX_VALID needs the `states` buffer that holds the arrays");
    if (a->states) {  // the per-position arrays live behind the tile states, kept for later calls on the same inputs
        tcum = (float*)((char*)a->states + tile_states_bytes(d));
        if (a->dt) dtT = tcum + (size_t)d.b * d.h * d.T;
        if (a->skip) skipT = tcum + 2 * (size_t)d.b * d.h * d.T;
        extreme = (int*)(tcum + 3 * (size_t)d.b * d.h * d.T);
        if (!aux_valid && cudaMemsetAsync(extreme, 0, 4, st) != cudaSuccess) SSD_TC_FAIL(SSD_B200_ECUDA, "memset failed");
    }
    if (cudaMemsetAsync(status, 0, 8, st) != cudaSuccess) SSD_TC_FAIL(SSD_B200_ECUDA, "memset failed");
    if (!a->cumsum_is_input && !aux_valid && d.l == LT) {
        // chunk = tile: the within-chunk cumulative sums, their log2 copies, the transposes and the flag in one kernel
        dim3 g(d.T / LT, (d.h + 31) / 32, d.b);
        if (a->skip)
            SSD_LAUNCH(prof::K_CUMSUM, st, (cumsum_tile_fused_kernel<64, true><<<g, 256, 0, st>>>(
                a->a, a->shape.a_dtype == SSD_B200_BF16, a->dt, a->A_head, a->a_cumsum, tcum, dtT, a->skip, skipT, extreme, d.T, d.h)));
        else
            SSD_LAUNCH(prof::K_CUMSUM, st, (cumsum_tile_fused_kernel<128, false><<<g, 256, 0, st>>>(
                a->a, a->shape.a_dtype == SSD_B200_BF16, a->dt, a->A_head, a->a_cumsum, tcum, dtT, nullptr, nullptr, extreme, d.T, d.h)));
        SSD_TC_CHECK("cumsum_tile_fused");
    } else {
        if (!a->cumsum_is_input) {
            simt::Params P{};
            P.d = d; P.a = a->a; P.dt = a->a ? nullptr : a->dt; P.A_head = a->A_head; P.cum = a->a_cumsum;
            P.a_is_bf16 = a->shape.a_dtype == SSD_B200_BF16;
            size_t sm = (size_t)d.l * (d.h + 1) * 4;
            if (sm > 48 * 1024 &&
                cudaFuncSetAttribute(simt::chunk_cumsum_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm) != cudaSuccess)
                SSD_TC_FAIL(SSD_B200_ECUDA, "chunk_cumsum: set shared memory size failed");
            SSD_LAUNCH(prof::K_CUMSUM, st, simt::chunk_cumsum_kernel<<<dim3(d.c, d.b), simt::NTHR, sm, st>>>(P));
            SSD_TC_CHECK("chunk_cumsum");
        }
        if (!aux_valid)
            if (int rc = launch_tile_cumsum(d, a->a_cumsum, a->dt, tcum, dtT, a->skip, skipT, extreme, st, err, errn)) return rc;
    }
    if (int rc = set_walk_attrs(err, errn)) return rc;
    WalkParams P{};
    P.skipT = skipT;
    P.extreme = extreme;
    P.ysq = a->ysq;
    const uint64_t rows = (uint64_t)d.b * d.T;
    bool ok = make_map(&P.mU, a->x, rows, (uint64_t)d.h * HP) && make_map(&P.mV, a->B, rows, (uint64_t)d.g * DN) &&
              make_map(&P.mC, a->C, rows, (uint64_t)d.g * DN) &&
              make_map(&P.mY, states_only ? a->x : (const void*)a->y, rows, (uint64_t)d.h * HP);
    if (a->states && ((uintptr_t)a->states & 15)) SSD_TC_FAIL(SSD_B200_EINVAL, "`states` must be 16-byte aligned");
    if (ok && a->states && !states_only) {
        ok = make_map(&P.mS, a->states, (uint64_t)d.b * (d.T / LT) * d.h * DN, HP);
        P.save_states = 1;
    } else {
        P.mS = P.mY;
    }
    if (!ok) SSD_TC_FAIL(SSD_B200_ECUDA, "tensor map encoding failed");
    P.tcum = tcum; P.dtT = dtT; P.D = a->D; P.seed = a->init; P.out_state = a->final_state; P.status = status;
    P.T = d.T; P.h = d.h; P.hpg = d.hpg; P.nt = d.T / LT;
    if (states_only) {  // what this piece of the sequence adds to the state after it (plus the decayed seed)
        SummaryParams S{};
        S.mU = P.mU; S.mV = P.mV; S.tcum = tcum; S.dtT = dtT; S.seed = a->init; S.out = a->final_state;
        S.logdecay = a->logdecay_total; S.status = status; S.T = d.T; S.h = d.h; S.hpg = d.hpg; S.nt = d.T / LT;
        if (d.hpg % 2 == 0)  // two heads of a group per CTA share the group's panels
            SSD_LAUNCH(prof::K_TC_SUMMARY, st, (summary_kernel<false, 2><<<dim3(d.h / 2, d.b), SumCfg<2>::THREADS, SumCfg<2>::SMEM, st>>>(S)));
        else
            SSD_LAUNCH(prof::K_TC_SUMMARY, st, (summary_kernel<false, 1><<<dim3(d.h, d.b), SumCfg<1>::THREADS, SumCfg<1>::SMEM, st>>>(S)));
        SSD_TC_CHECK("tc_summary_fwd");
        return 0;
    }
    SSD_LAUNCH(prof::K_TC_FWD, st, (fwd_walk_kernel<false><<<dim3(d.h, d.b), kFwdThreads, kFwdSmem, st>>>(P)));
    SSD_LAUNCH(prof::K_TC_FWD_ALT, st, (fwd_walk_kernel<true><<<dim3(d.h, d.b), kFwdThreads, kFwdSmem, st>>>(P)));
    SSD_TC_CHECK("tc_fwd_walk");
    if (a->logdecay_total) {
        SSD_LAUNCH(prof::K_CUMSUM, st, simt::logdecay_total_kernel<<<(d.b * d.h + 127) / 128, 128, 0, st>>>(a->a_cumsum, a->logdecay_total, d.b * d.h, d.c, d.l));
        SSD_TC_CHECK("logdecay_total");
    }
    return 0;
}

inline int backward(const ssd_b200_bwd_args* a, const Dims& d, cudaStream_t st, char* err, size_t errn) {
    Ws w = ws_layout(d, SSD_B200_PASS_BWD);
    if (a->workspace_bytes < w.total) SSD_TC_FAIL(SSD_B200_EWORKSPACE, "workspace %zu < %zu", a->workspace_bytes, w.total);
    if (!encode_fn()) SSD_TC_FAIL(SSD_B200_ECUDA, "cuTensorMapEncodeTiled is not available");
    for (const void* p : {a->x, a->B, a->C, a->dy, (const void*)a->dx, (const void*)a->dB, (const void*)a->dC})
        if ((uintptr_t)p & 15) SSD_TC_FAIL(SSD_B200_EINVAL, "tensor-core path needs 16-byte aligned tensors");
    char* ws = (char*)a->workspace;
    int* status = (int*)(ws + w.status);
    float* tcum = (float*)(ws + w.tcum);
    float* dtT = a->dt ? (float*)(ws + w.dtT) : nullptr;
    const void* Hst = a->states ? a->states : (const void*)(ws + w.Hst);
    if ((uintptr_t)Hst & 15) SSD_TC_FAIL(SSD_B200_EINVAL, "`states` must be 16-byte aligned");
    void* Qst = ws + w.Qst;
    float* fin = (float*)(ws + w.final_state);
    float* dinit = a->dinit ? a->dinit : (float*)(ws + w.dinit);
    if (cudaMemsetAsync(status, 0, 8, st) != cudaSuccess) SSD_TC_FAIL(SSD_B200_ECUDA, "memset failed");
    int* extreme = status + 1;
    float* skipT = a->skip ? (float*)(ws + w.skipT) : nullptr;
    if (a->states) {  // the forward left the arrays and the flag behind the tile states
        tcum = (float*)((uintptr_t)a->states + tile_states_bytes(d));
        dtT = a->dt ? tcum + (size_t)d.b * d.h * d.T : nullptr;
        skipT = a->skip ? tcum + 2 * (size_t)d.b * d.h * d.T : nullptr;
        extreme = (int*)(tcum + 3 * (size_t)d.b * d.h * d.T);
    } else if (int rc = launch_tile_cumsum(d, a->a_cumsum, a->dt, tcum, dtT, a->skip, skipT, extreme, st, err, errn)) {
        return rc;
    }
    if (int rc = set_walk_attrs(err, errn)) return rc;
    const int nt = d.T / LT;
    const uint64_t rows = (uint64_t)d.b * d.T, srows = (uint64_t)d.b * nt * d.h * DN;
    if (a->flags & SSD_B200_BWD_DINIT_ONLY) {  // d(initial state) of this piece for the given (or a zero) dfinal
        SummaryParams S{};
        if (!(make_map(&S.mU, a->dy, rows, (uint64_t)d.h * HP) && make_map(&S.mV, a->C, rows, (uint64_t)d.g * DN)))
            SSD_TC_FAIL(SSD_B200_ECUDA, "tensor map encoding failed");
        S.tcum = tcum; S.dtT = nullptr; S.seed = a->dfinal; S.out = a->dinit; S.logdecay = nullptr; S.status = status;
        S.T = d.T; S.h = d.h; S.hpg = d.hpg; S.nt = nt;
        if (d.hpg % 2 == 0)
            SSD_LAUNCH(prof::K_TC_SUMMARY, st, (summary_kernel<true, 2><<<dim3(d.h / 2, d.b), SumCfg<2>::THREADS, SumCfg<2>::SMEM, st>>>(S)));
        else
            SSD_LAUNCH(prof::K_TC_SUMMARY, st, (summary_kernel<true, 1><<<dim3(d.h, d.b), SumCfg<1>::THREADS, SumCfg<1>::SMEM, st>>>(S)));
        SSD_TC_CHECK("tc_summary_rev");
        return 0;
    }
    CUtensorMap mX, mdY, mB, mC, mH, mQ, mdX, mdB, mdC;
    bool ok = make_map(&mX, a->x, rows, (uint64_t)d.h * HP) && make_map(&mdY, a->dy, rows, (uint64_t)d.h * HP) &&
              make_map(&mB, a->B, rows, (uint64_t)d.g * DN) && make_map(&mC, a->C, rows, (uint64_t)d.g * DN) &&
              make_map(&mH, Hst, srows, HP) && make_map(&mQ, Qst, srows, HP) &&
              make_map(&mdX, a->dx, rows, (uint64_t)d.h * HP) && make_map(&mdB, a->dB, rows, (uint64_t)d.g * DN) &&
              make_map(&mdC, a->dC, rows, (uint64_t)d.g * DN);
    if (!ok) SSD_TC_FAIL(SSD_B200_ECUDA, "tensor map encoding failed");
    if (!a->states) {  // states entering every tile (skipped when the forward saved them)
        WalkParams P{};
        P.mU = mX; P.mV = mB; P.mC = mC; P.mY = mdX; P.mS = mH; P.save_states = 1;
        P.tcum = tcum; P.dtT = dtT; P.D = nullptr; P.seed = a->init; P.out_state = fin; P.status = status;
        P.T = d.T; P.h = d.h; P.hpg = d.hpg; P.nt = nt;
        SSD_LAUNCH(prof::K_TC_BWD_STATE, st, (states_walk_kernel<<<dim3(d.h, d.b), kWalkThreads, WalkCfg<1>::SMEM, st>>>(P)));
        SSD_TC_CHECK("tc_bwd_state");
    }
    {   // reverse walk: gradient of the state leaving every tile, and d(initial state)
        WalkParams P{};
        P.mU = mdY; P.mV = mC; P.mC = mC; P.mY = mdX; P.mS = mQ; P.save_states = 1;
        P.tcum = tcum; P.dtT = nullptr; P.D = nullptr; P.seed = a->dfinal; P.out_state = dinit; P.status = status;
        P.T = d.T; P.h = d.h; P.hpg = d.hpg; P.nt = nt;
        if (d.hpg % 2 == 0)  // two heads of a group per CTA: shared C panels, one N = 128 product per tile
            SSD_LAUNCH(prof::K_TC_BWD_STATE, st, rev_walk_kernel<2><<<dim3(d.h / 2, d.b), RevCfg<2>::THREADS, RevCfg<2>::SMEM, st>>>(P));
        else
            SSD_LAUNCH(prof::K_TC_BWD_STATE, st, rev_walk_kernel<1><<<dim3(d.h, d.b), RevCfg<1>::THREADS, RevCfg<1>::SMEM, st>>>(P));
        SSD_TC_CHECK("tc_bwd_dstate");
    }
    {
        BwdParams P{};
        P.mX = mX; P.mdY = mdY; P.mB = mB; P.mC = mC; P.mH = mH; P.mQ = mQ; P.mdX = mdX; P.mdB = mdB; P.mdC = mdC;
        P.tcum = tcum; P.dtT = dtT; P.D = a->D; P.skipT = skipT; P.g = (float*)(ws + w.g); P.ddtx = (float*)(ws + w.ddtx);
        P.dyx = (float*)(ws + w.dyx); P.status = status; P.T = d.T; P.h = d.h;
        P.hpg = d.hpg; P.nt = nt; P.b = d.b; P.gS = (float*)(ws + w.gS);
        P.items = nt * d.g * d.b;
        P.extreme = extreme;
        const dim3 grid(std::min(P.items, sm_count()));
        SSD_LAUNCH(prof::K_TC_BWD, st, bwd_tile_kernel<false><<<grid, kBwdThreads, kBwdSmem, st>>>(P));
        SSD_LAUNCH(prof::K_TC_BWD_ALT, st, bwd_tile_kernel<true><<<grid, kBwdThreads, kBwdSmem, st>>>(P));
        SSD_TC_CHECK("tc_bwd_walk");
    }
    {
        DecayTileParams P{};
        P.g = (const float*)(ws + w.g); P.ddtx = (const float*)(ws + w.ddtx); P.gS = (const float*)(ws + w.gS);
        P.dyx = (a->dt && (a->D || a->skip)) ? (const float*)(ws + w.dyx) : nullptr;
        P.dt = a->dt; P.A_head = a->A_head; P.ddt = a->ddt; P.da = a->cumsum_is_input ? nullptr : a->da;
        P.dskip = a->skip ? a->dskip : nullptr;
        P.dAh_part = (float*)(ws + w.dAh_part); P.dD_part = P.dyx ? (float*)(ws + w.dD_part) : nullptr;
        P.b = d.b; P.T = d.T; P.h = d.h; P.nt = nt;
        SSD_LAUNCH(prof::K_DECAY, st, decay_tile_kernel<<<dim3(nt, (d.h + 31) / 32, d.b), 256, 0, st>>>(P));
        SSD_TC_CHECK("decay_grad");
        if (a->dt && a->A_head) {
            SSD_LAUNCH(prof::K_REDUCE, st, reduce_rows_kernel<<<dim3(d.h, a->D ? 2 : 1), 256, 0, st>>>(
                P.dAh_part, a->dA_head, d.b * nt, d.h, P.dD_part, a->dD));
            SSD_TC_CHECK("reduce_batch");
        }
    }
    return 0;
}

}  // namespace tc
}  // namespace ssd
