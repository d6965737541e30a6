// C-ABI entry points of the SSD chunked scan library: argument validation, workspace
// carving and kernel dispatch.  See include/ssd_b200.h for the contract.
#include "../../include/ssd_b200.h"

#include <cstdarg>
#include <cstdio>
#include <cstring>

#include "ssd_simt.cuh"
#include "ssd_tc_host.cuh"
#include "ssd_mamba3.cuh"
#include "ssd_elementwise.cuh"

#include <atomic>
#include <vector>

namespace ssd {
namespace prof {
// Launch accounting and optional per-kernel CUDA-event timing (benchmark use, one host thread).
const char* const kNames[K_COUNT] = {
    "chunk_cumsum", "chunk_state", "state_passing", "chunk_scan", "chunk_dstate", "state_passing_rev",
    "bwd_row", "bwd_col", "decay_grad", "reduce_batch", "cache_L", "cache_decay_chunk", "state_prefix",
    "tc_fwd_walk", "tc_bwd_state", "tc_bwd_walk", "tc_aux", "tc_summary", "tc_bwd_walk_alt", "tc_fwd_walk_alt", "exchange"};
std::atomic<long long> g_launches{0};
bool g_enabled = false;
struct Rec {
    int k;
    cudaEvent_t a, b;
};
std::vector<Rec> g_recs;
void begin(int k, cudaStream_t st) {
    g_launches.fetch_add(1, std::memory_order_relaxed);
    if (!g_enabled) return;
    Rec r{k, nullptr, nullptr};
    if (cudaEventCreate(&r.a) != cudaSuccess || cudaEventCreate(&r.b) != cudaSuccess) return;
    cudaEventRecord(r.a, st);
    g_recs.push_back(r);
}
void end(cudaStream_t st) {
    if (!g_enabled || g_recs.empty()) return;
    cudaEventRecord(g_recs.back().b, st);
}
}  // namespace prof
}  // namespace ssd

namespace {

thread_local char g_err[512] = "";

int fail(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
    return code;
}

size_t align_up(size_t v, size_t a = 256) { return (v + a - 1) / a * a; }

int check_shape(const ssd_b200_shape* s) {
    if (!s) return fail(SSD_B200_EINVAL, "shape is null");
    if (s->abi_version != SSD_B200_ABI_VERSION)
        return fail(SSD_B200_EINVAL, "abi_version %d != %d", s->abi_version, SSD_B200_ABI_VERSION);
    if (s->dtype != SSD_B200_F32 && s->dtype != SSD_B200_BF16) return fail(SSD_B200_EINVAL, "bad dtype %d", s->dtype);
    if (s->a_dtype != SSD_B200_F32 && s->a_dtype != SSD_B200_BF16)
        return fail(SSD_B200_EINVAL, "bad a_dtype %d", s->a_dtype);
    if (s->batch <= 0 || s->seqlen <= 0 || s->nheads <= 0 || s->headdim <= 0 || s->dstate <= 0 || s->ngroups <= 0 ||
        s->chunk <= 0)
        return fail(SSD_B200_EINVAL, "non-positive dimension");
    if (s->seqlen % s->chunk != 0)
        return fail(SSD_B200_EINVAL, "sequence length %lld not divisible by chunk_size %lld", (long long)s->seqlen,
                    (long long)s->chunk);
    if (s->nheads % s->ngroups != 0)
        return fail(SSD_B200_EINVAL, "nheads %lld not divisible by ngroups %lld", (long long)s->nheads,
                    (long long)s->ngroups);
    if (s->batch * (s->seqlen / s->chunk) > 65535 * 32 || s->batch > 65535 || s->nheads > 65535)
        return fail(SSD_B200_EUNSUPPORTED, "grid dimension too large");
    if ((double)s->batch * s->seqlen * s->nheads * s->headdim > 2.0e18) return fail(SSD_B200_EINVAL, "size overflow");
    if (s->path < SSD_B200_PATH_AUTO || s->path > SSD_B200_PATH_TC) return fail(SSD_B200_EINVAL, "bad path %d", s->path);
    return 0;
}

ssd::Dims dims_of(const ssd_b200_shape& s) {
    ssd::Dims d;
    d.b = (int)s.batch;
    d.T = (int)s.seqlen;
    d.h = (int)s.nheads;
    d.p = (int)s.headdim;
    d.n = (int)s.dstate;
    d.g = (int)s.ngroups;
    d.l = (int)s.chunk;
    d.c = d.T / d.l;
    d.hpg = d.h / d.g;
    return d;
}

bool simt_supported(const ssd_b200_shape& s, const char** why) {
    if (s.headdim > 128) {
        *why = "SIMT path needs headdim <= 128";
        return false;
    }
    if (s.dstate > 256) {
        *why = "SIMT path needs d_state <= 256";
        return false;
    }
    if (s.batch * (s.seqlen / s.chunk) > 65535) {
        *why = "SIMT path needs batch * nchunks <= 65535";
        return false;
    }
    if (s.chunk > 1024 || s.chunk * (s.nheads + 1) * 4 > 200 * 1024) {
        *why = "SIMT path: chunk * nheads too large for the cumsum tile";
        return false;
    }
    return true;
}

int resolve_path(const ssd_b200_shape& s) {
    const char* why = "";
    const bool tc = ssd::tc::supported(s.dtype, (int)s.seqlen, (int)s.nheads, (int)s.headdim, (int)s.dstate,
                                       (int)s.ngroups, (int)s.chunk);
    if (s.path == SSD_B200_PATH_TC) {
        if (!tc) return fail(SSD_B200_EUNSUPPORTED, "tensor-core path does not cover this shape/dtype");
        return SSD_B200_PATH_TC;
    }
    if (s.path == SSD_B200_PATH_AUTO && tc) return SSD_B200_PATH_TC;
    if (!simt_supported(s, &why)) return fail(SSD_B200_EUNSUPPORTED, "%s", why);
    return SSD_B200_PATH_SIMT;
}

// Workspace layout of the SIMT path (all fp32, each block 256-byte aligned).
struct SimtWs {
    size_t states, dstates, final_state, g_row, g_col, ddtx, dAh_part, dD_part, dinit, total;
};

SimtWs simt_ws(const ssd::Dims& d, int pass) {
    SimtWs w{};
    size_t off = 0;
    const size_t st = (size_t)d.b * d.c * d.h * d.p * d.n * 4;
    const size_t bhpn = (size_t)d.b * d.h * d.p * d.n * 4;
    const size_t bht = (size_t)d.b * d.h * d.T * 4;
    const size_t bh = (size_t)d.b * d.h * 4;
    auto take = [&](size_t bytes) {
        size_t o = off;
        off += align_up(bytes);
        return o;
    };
    w.states = take(st);
    if (pass == SSD_B200_PASS_BWD) {
        w.dstates = take(st);
        w.final_state = take(bhpn);
        w.dinit = take(bhpn);
        w.g_row = take(bht);
        w.g_col = take(bht);
        w.ddtx = take(bht);
        w.dAh_part = take(bh);
        w.dD_part = take(bh);
    }
    w.total = off;
    return w;
}

#define CUDA_LAUNCH_CHECK(what)                                                              \
    do {                                                                                     \
        cudaError_t e_ = cudaGetLastError();                                                 \
        if (e_ != cudaSuccess) return fail(SSD_B200_ECUDA, "%s: %s", what, cudaGetErrorString(e_)); \
    } while (0)

template <class K>
int set_smem(K kernel, size_t bytes, const char* name) {
    if (bytes > 227 * 1024) return fail(SSD_B200_EUNSUPPORTED, "%s needs %zu bytes of shared memory", name, bytes);
    if (bytes > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
        if (e != cudaSuccess) return fail(SSD_B200_ECUDA, "%s: set smem: %s", name, cudaGetErrorString(e));
    }
    return 0;
}

template <class T>
int simt_forward_states(const ssd::simt::Params& P, cudaStream_t st) {
    using namespace ssd::simt;
    const ssd::Dims& d = P.d;
    dim3 gs((d.n + TS - 1) / TS, (d.p + TS - 1) / TS, d.b * d.c * d.h);
    SSD_LAUNCH(ssd::prof::K_CHUNK_STATE, st, chunk_state_kernel<T><<<gs, NTHR, 0, st>>>(P, 0));
    CUDA_LAUNCH_CHECK("chunk_state");
    const size_t pn = (size_t)d.p * d.n;
    dim3 gp((unsigned)((pn + NTHR - 1) / NTHR), d.h, d.b);
    SSD_LAUNCH(ssd::prof::K_STATE_PASS, st, state_passing_kernel<<<gp, NTHR, 0, st>>>(P, 0));
    CUDA_LAUNCH_CHECK("state_passing");
    return 0;
}

int launch_cumsum(const ssd::simt::Params& P, cudaStream_t st) {
    using namespace ssd::simt;
    const ssd::Dims& d = P.d;
    size_t sm = (size_t)d.l * (d.h + 1) * 4;
    if (int rc = set_smem(chunk_cumsum_kernel, sm, "chunk_cumsum")) return rc;
    SSD_LAUNCH(ssd::prof::K_CUMSUM, st, chunk_cumsum_kernel<<<dim3(d.c, d.b), NTHR, sm, st>>>(P));
    CUDA_LAUNCH_CHECK("chunk_cumsum");
    return 0;
}

template <class T>
int simt_fwd(const ssd_b200_fwd_args* a, cudaStream_t st) {
    using namespace ssd::simt;
    Params P{};
    P.d = dims_of(a->shape);
    const ssd::Dims& d = P.d;
    SimtWs w = simt_ws(d, SSD_B200_PASS_FWD);
    if (a->workspace_bytes < w.total) return fail(SSD_B200_EWORKSPACE, "workspace %zu < %zu", a->workspace_bytes, w.total);
    char* ws = (char*)a->workspace;
    P.x = a->x; P.a = a->a; P.dt = a->dt; P.A_head = a->A_head; P.D = a->D; P.B = a->B; P.C = a->C;
    P.init = a->init; P.cum = a->a_cumsum; P.states = (float*)(ws + w.states);
    P.final_state = a->final_state; P.y = a->y; P.a_is_bf16 = a->shape.a_dtype == SSD_B200_BF16;
    if (!a->cumsum_is_input)
        if (int rc = launch_cumsum(P, st)) return rc;
    if (int rc = simt_forward_states<T>(P, st)) return rc;
    if (a->logdecay_total) {
        SSD_LAUNCH(ssd::prof::K_CUMSUM, st, logdecay_total_kernel<<<(d.b * d.h + 127) / 128, 128, 0, st>>>(a->a_cumsum, a->logdecay_total, d.b * d.h, d.c, d.l));
        CUDA_LAUNCH_CHECK("logdecay_total");
    }
    if (a->flags & SSD_B200_FWD_STATES_ONLY) return 0;
    const int PT = (d.p + TS - 1) / TS;
    const int hrows = d.p > TS ? d.p : TS;
    size_t sm = ((size_t)TS * (d.n + 1) + (size_t)hrows * (d.n + 1) + (size_t)TS * (PT * TS + 1) + TS * (TS + 1) + 2 * TS) * 4;
    dim3 g((d.l + TS - 1) / TS, d.h, d.b * d.c);
    if (PT == 1) {
        if (int rc = set_smem(chunk_scan_kernel<T, 1>, sm, "chunk_scan")) return rc;
        SSD_LAUNCH(ssd::prof::K_CHUNK_SCAN, st, chunk_scan_kernel<T, 1><<<g, NTHR, sm, st>>>(P));
    } else {
        if (int rc = set_smem(chunk_scan_kernel<T, 2>, sm, "chunk_scan")) return rc;
        SSD_LAUNCH(ssd::prof::K_CHUNK_SCAN, st, chunk_scan_kernel<T, 2><<<g, NTHR, sm, st>>>(P));
    }
    CUDA_LAUNCH_CHECK("chunk_scan");
    return 0;
}

template <class T, int NTN>
int launch_bwd_row(const ssd::simt::Params& P, cudaStream_t st) {
    using namespace ssd::simt;
    const ssd::Dims& d = P.d;
    const int hrows = d.p > TS ? d.p : TS;
    const int pp_pad = (d.p + 3) / 4 * 4;
    size_t sm = ((size_t)TS * (d.n + 1) + (size_t)hrows * (d.n + 1) + 2 * (size_t)TS * (pp_pad + 1) + TS * (TS + 1) + 2 * TS) * 4;
    if (int rc = set_smem(bwd_row_kernel<T, NTN>, sm, "bwd_row")) return rc;
    SSD_LAUNCH(ssd::prof::K_BWD_ROW, st, bwd_row_kernel<T, NTN><<<dim3((d.l + TS - 1) / TS, d.g, d.b * d.c), NTHR, sm, st>>>(P));
    CUDA_LAUNCH_CHECK("bwd_row");
    return 0;
}

template <class T, int NTN, int PT>
int launch_bwd_col(const ssd::simt::Params& P, cudaStream_t st) {
    using namespace ssd::simt;
    const ssd::Dims& d = P.d;
    const int hrows = d.p > TS ? d.p : TS;
    size_t sm = ((size_t)TS * (d.n + 1) + (size_t)hrows * (d.n + 1) + 2 * (size_t)TS * (PT * TS + 1) + 2 * TS * (TS + 1) + 3 * TS) * 4;
    if (int rc = set_smem(bwd_col_kernel<T, NTN, PT>, sm, "bwd_col")) return rc;
    SSD_LAUNCH(ssd::prof::K_BWD_COL, st, bwd_col_kernel<T, NTN, PT><<<dim3((d.l + TS - 1) / TS, d.g, d.b * d.c), NTHR, sm, st>>>(P));
    CUDA_LAUNCH_CHECK("bwd_col");
    return 0;
}

template <class T>
int simt_bwd(const ssd_b200_bwd_args* a, cudaStream_t st) {
    using namespace ssd::simt;
    Params P{};
    P.d = dims_of(a->shape);
    const ssd::Dims& d = P.d;
    SimtWs w = simt_ws(d, SSD_B200_PASS_BWD);
    if (a->workspace_bytes < w.total) return fail(SSD_B200_EWORKSPACE, "workspace %zu < %zu", a->workspace_bytes, w.total);
    char* ws = (char*)a->workspace;
    P.x = a->x; P.a = a->a; P.dt = a->dt; P.A_head = a->A_head; P.D = a->D; P.B = a->B; P.C = a->C;
    P.dy = a->dy; P.init = a->init; P.dfinal = a->dfinal; P.cum = (float*)a->a_cumsum;
    P.states = (float*)(ws + w.states); P.dstates = (float*)(ws + w.dstates);
    P.final_state = (float*)(ws + w.final_state);
    P.dinit = a->dinit ? a->dinit : (float*)(ws + w.dinit);
    P.dx = a->dx; P.dB = a->dB; P.dC = a->dC;
    P.g_row = (float*)(ws + w.g_row); P.g_col = (float*)(ws + w.g_col); P.ddtx = (float*)(ws + w.ddtx);
    P.da = a->cumsum_is_input ? nullptr : a->da;
    P.ddt = a->ddt; P.dAh_part = (float*)(ws + w.dAh_part); P.dD_part = (float*)(ws + w.dD_part);
    P.a_is_bf16 = a->shape.a_dtype == SSD_B200_BF16;
    const bool dinit_only = (a->flags & SSD_B200_BWD_DINIT_ONLY) != 0;
    // states entering each chunk (recomputed) and the final state
    if (!dinit_only)
        if (int rc = simt_forward_states<T>(P, st)) return rc;
    // local state gradients and the reverse recurrence
    dim3 gs((d.n + TS - 1) / TS, (d.p + TS - 1) / TS, d.b * d.c * d.h);
    SSD_LAUNCH(ssd::prof::K_CHUNK_DSTATE, st, chunk_state_kernel<T><<<gs, NTHR, 0, st>>>(P, 1));
    CUDA_LAUNCH_CHECK("chunk_dstate");
    const size_t pn = (size_t)d.p * d.n;
    SSD_LAUNCH(ssd::prof::K_STATE_PASS_REV, st, state_passing_kernel<<<dim3((unsigned)((pn + NTHR - 1) / NTHR), d.h, d.b), NTHR, 0, st>>>(P, 1));
    CUDA_LAUNCH_CHECK("state_passing_rev");
    if (dinit_only) return 0;
    const int NTN = (d.n + TS - 1) / TS, PT = (d.p + TS - 1) / TS;
    int rc = 0;
    if (NTN <= 1) rc = launch_bwd_row<T, 1>(P, st);
    else if (NTN == 2) rc = launch_bwd_row<T, 2>(P, st);
    else rc = launch_bwd_row<T, 4>(P, st);
    if (rc) return rc;
    if (PT == 1) {
        if (NTN <= 1) rc = launch_bwd_col<T, 1, 1>(P, st);
        else if (NTN == 2) rc = launch_bwd_col<T, 2, 1>(P, st);
        else rc = launch_bwd_col<T, 4, 1>(P, st);
    } else {
        if (NTN <= 1) rc = launch_bwd_col<T, 1, 2>(P, st);
        else if (NTN == 2) rc = launch_bwd_col<T, 2, 2>(P, st);
        else rc = launch_bwd_col<T, 4, 2>(P, st);
    }
    if (rc) return rc;
    SSD_LAUNCH(ssd::prof::K_DECAY, st, decay_grad_kernel<T><<<dim3(d.h, d.b), NTHR, 0, st>>>(P));
    CUDA_LAUNCH_CHECK("decay_grad");
    if (a->dt) {
        SSD_LAUNCH(ssd::prof::K_REDUCE, st, reduce_batch_kernel<<<(d.h + 127) / 128, 128, 0, st>>>(P.dAh_part, a->dA_head, d.b, d.h));
        if (a->D) SSD_LAUNCH(ssd::prof::K_REDUCE, st, reduce_batch_kernel<<<(d.h + 127) / 128, 128, 0, st>>>(P.dD_part, a->dD, d.b, d.h));
        CUDA_LAUNCH_CHECK("reduce_batch");
    }
    return 0;
}

// 1 = operator form (a), 2 = Mamba-2 form (dt, A_head[, D]), 3 = scaled operator form (a and dt[, skip]); < 0 = error
int check_forms(const void* a, const float* dt, const float* A_head, const float* D, const float* skip) {
    if (a && dt) {
        if (A_head || D) return fail(SSD_B200_EINVAL, "scaled operator form takes a and dt (and skip), not A_head or D");
        return 3;
    }
    if (skip) return fail(SSD_B200_EINVAL, "skip belongs to the scaled operator form (a and dt both given)");
    if (a) {
        if (A_head || D) return fail(SSD_B200_EINVAL, "give either a, or dt and A_head (and D), not both");
        return 1;
    }
    if (!dt || !A_head) return fail(SSD_B200_EINVAL, "need a, or both dt and A_head");
    return 2;
}

}  // namespace

namespace {
// Threads per (b,t,h) row of the trapezoid kernels: p / V when that is a power of two <= 32 (16-byte accesses),
// else 0 = scalar fallback with a full warp per row.
template <class T>
int m3_row_threads(int p) {
    constexpr int V = ssd::m3::VecOf<T>::N;
    if (p % V) return 0;
    const int tpr = p / V;
    return (tpr <= 32 && (tpr & (tpr - 1)) == 0) ? tpr : 0;
}
#define M3_ROW_DISPATCH(KERNEL, ...)                                                                              \
    do {                                                                                                          \
        constexpr int V = ssd::m3::VecOf<T>::N;                                                                   \
        const int tpr = m3_row_threads<T>(d.p);                                                                   \
        const size_t thr = rows * (size_t)(tpr ? tpr : 32);                                                       \
        const unsigned blocks = (unsigned)((thr + 255) / 256);                                                    \
        switch (tpr) {                                                                                            \
            case 1: SSD_LAUNCH(ssd::prof::K_TC_AUX, st, (KERNEL<T, V, 1><<<blocks, 256, 0, st>>>(__VA_ARGS__))); break;   \
            case 2: SSD_LAUNCH(ssd::prof::K_TC_AUX, st, (KERNEL<T, V, 2><<<blocks, 256, 0, st>>>(__VA_ARGS__))); break;   \
            case 4: SSD_LAUNCH(ssd::prof::K_TC_AUX, st, (KERNEL<T, V, 4><<<blocks, 256, 0, st>>>(__VA_ARGS__))); break;   \
            case 8: SSD_LAUNCH(ssd::prof::K_TC_AUX, st, (KERNEL<T, V, 8><<<blocks, 256, 0, st>>>(__VA_ARGS__))); break;   \
            case 16: SSD_LAUNCH(ssd::prof::K_TC_AUX, st, (KERNEL<T, V, 16><<<blocks, 256, 0, st>>>(__VA_ARGS__))); break; \
            case 32: SSD_LAUNCH(ssd::prof::K_TC_AUX, st, (KERNEL<T, V, 32><<<blocks, 256, 0, st>>>(__VA_ARGS__))); break; \
            default: SSD_LAUNCH(ssd::prof::K_TC_AUX, st, (KERNEL<T, 1, 32><<<blocks, 256, 0, st>>>(__VA_ARGS__))); break; \
        }                                                                                                         \
    } while (0)

template <class T>
int m3_fwd_impl(const ssd::Dims& d, const void* x, const float* dt, const float* lam, const float* A_head, const void* B,
                const void* C, const void* ang, bool ang_f32, void* xw, float* dA, void* Br, void* Cr, float* sdot, float* cum,
                float* segsum, const float* D, float* wout, float* skip, cudaStream_t st) {
    using namespace ssd::m3;
    const int E = d.h * (d.n / 2), nseg = (d.T + SEG - 1) / SEG;
    dim3 gs(nseg, (E + 255) / 256, d.b);
    if (ang_f32) {  // angles keep their own precision whatever the storage type of x, B and C
        SSD_LAUNCH(ssd::prof::K_TC_AUX, st, scanT_segsum_kernel<float><<<gs, 256, 0, st>>>((const float*)ang, segsum, d.T, E));
        SSD_LAUNCH(ssd::prof::K_TC_AUX, st, (scanT_apply_kernel<float, float><<<gs, 256, 0, st>>>((const float*)ang, segsum, cum, d.T, E, 0, -1.f)));
    } else {
        SSD_LAUNCH(ssd::prof::K_TC_AUX, st, scanT_segsum_kernel<T><<<gs, 256, 0, st>>>((const T*)ang, segsum, d.T, E));
        SSD_LAUNCH(ssd::prof::K_TC_AUX, st, (scanT_apply_kernel<T, float><<<gs, 256, 0, st>>>((const T*)ang, segsum, cum, d.T, E, 0, -1.f)));
    }
    if (d.n % VecOf<T>::N == 0)
        SSD_LAUNCH(ssd::prof::K_TC_AUX, st, (rope_fwd_kernel<T, VecOf<T>::N><<<dim3(d.T, d.b), 256, 0, st>>>((const T*)B, (const T*)C, cum, (T*)Br, (T*)Cr, d.T, d.h, d.g, d.n)));
    else
        SSD_LAUNCH(ssd::prof::K_TC_AUX, st, (rope_fwd_kernel<T, 2><<<dim3(d.T, d.b), 256, 0, st>>>((const T*)B, (const T*)C, cum, (T*)Br, (T*)Cr, d.T, d.h, d.g, d.n)));
    const size_t grows = (size_t)d.b * d.T * d.g, rows = (size_t)d.b * d.T * d.h;
    SSD_LAUNCH(ssd::prof::K_TC_AUX, st, bc_dot_kernel<T><<<(unsigned)((grows + 7) / 8), 256, 0, st>>>((const T*)B, (const T*)C, sdot, d.n, grows));
    if (xw) {
        M3_ROW_DISPATCH(xw_fwd_kernel, (const T*)x, dt, lam, A_head, (T*)xw, dA, d.T, d.h, d.p, rows);
    } else {  // the scan takes the weight and the skip coefficient per position: x is not touched here
        SSD_LAUNCH(ssd::prof::K_TC_AUX, st, coef_fwd_kernel<<<(unsigned)((rows + 255) / 256), 256, 0, st>>>(dt, lam, A_head, D, sdot, wout, dA, skip, d.T, d.h, d.hpg, rows));
    }
    CUDA_LAUNCH_CHECK("mamba3 prologue forward");
    return 0;
}

template <class T>
int m3_skip_impl(const ssd::Dims& d, const void* y_scan, const void* x, const float* D, const float* dt, const float* lam,
                 const float* sdot, void* y, cudaStream_t st) {
    using namespace ssd::m3;
    const size_t rows = (size_t)d.b * d.T * d.h;
    M3_ROW_DISPATCH(skip_fwd_kernel, (const T*)y_scan, (const T*)x, D, dt, lam, sdot, (T*)y, d.T, d.h, d.hpg, d.p, rows);
    CUDA_LAUNCH_CHECK("mamba3 skip forward");
    return 0;
}

template <class T>
int m3_bwd_impl(const ssd::Dims& d, const void* x, const void* dy, const float* dt, const float* lam, const float* D,
                const void* B, const void* C, const float* cum, const float* sdot, const void* dxw, const void* dBr,
                const void* dCr, void* dx, float* dw, float* dyx, void* dB, void* dC, void* dang, bool ang_f32, float* dcum,
                float* segsum, cudaStream_t st) {
    using namespace ssd::m3;
    const int E = d.h * (d.n / 2), nseg = (d.T + SEG - 1) / SEG;
    const size_t rows = (size_t)d.b * d.T * d.h;
    if (dxw)  // otherwise the scan's backward has already produced dx, dw and dyx (scaled operator form)
        M3_ROW_DISPATCH(xw_bwd_kernel, (const T*)x, (const T*)dy, (const T*)dxw, dt, lam, D, sdot, (T*)dx, dw, dyx, d.T, d.h, d.hpg, d.p, rows);
    if (d.n % VecOf<T>::N == 0) {
        const size_t items = (size_t)d.b * d.T * d.g * (d.n / VecOf<T>::N);
        SSD_LAUNCH(ssd::prof::K_TC_AUX, st, (rope_bwd_kernel<T, VecOf<T>::N><<<(unsigned)((items + 255) / 256), 256, 0, st>>>((const T*)B, (const T*)C, cum, (const T*)dBr, (const T*)dCr, dyx, dt, lam, (T*)dB, (T*)dC, dcum, d.T, d.h, d.g, d.n, items)));
    } else {
        const size_t items = (size_t)d.b * d.T * d.g * (d.n / 2);
        SSD_LAUNCH(ssd::prof::K_TC_AUX, st, (rope_bwd_kernel<T, 2><<<(unsigned)((items + 255) / 256), 256, 0, st>>>((const T*)B, (const T*)C, cum, (const T*)dBr, (const T*)dCr, dyx, dt, lam, (T*)dB, (T*)dC, dcum, d.T, d.h, d.g, d.n, items)));
    }
    dim3 gs(nseg, (E + 255) / 256, d.b);
    SSD_LAUNCH(ssd::prof::K_TC_AUX, st, scanT_segsum_kernel<float><<<gs, 256, 0, st>>>(dcum, segsum, d.T, E));
    // d raw_angles[t] = - sum_{s >= t} d cum[s]
    if (ang_f32)
        SSD_LAUNCH(ssd::prof::K_TC_AUX, st, (scanT_apply_kernel<float, float><<<gs, 256, 0, st>>>(dcum, segsum, (float*)dang, d.T, E, 1, -1.f)));
    else
        SSD_LAUNCH(ssd::prof::K_TC_AUX, st, (scanT_apply_kernel<float, T><<<gs, 256, 0, st>>>(dcum, segsum, (T*)dang, d.T, E, 1, -1.f)));
    CUDA_LAUNCH_CHECK("mamba3 prologue backward");
    return 0;
}

template <class T>
int rope_op_impl(bool backward, long long BT, int H, int D, int aH, const void* x, const float* ang, const void* dy,
                 void* out, float* dang, cudaStream_t st) {
    using namespace ssd::ew;
    constexpr int V = VecOf<T>::N;
    const bool vec = D % V == 0;
    if (!backward) {
        if (vec) SSD_LAUNCH(ssd::prof::K_TC_AUX, st, (rope_op_fwd_kernel<T, V><<<(unsigned)BT, 256, 0, st>>>((const T*)x, ang, (T*)out, H, D, aH)));
        else SSD_LAUNCH(ssd::prof::K_TC_AUX, st, (rope_op_fwd_kernel<T, 2><<<(unsigned)BT, 256, 0, st>>>((const T*)x, ang, (T*)out, H, D, aH)));
    } else {
        if (vec) SSD_LAUNCH(ssd::prof::K_TC_AUX, st, (rope_op_bwd_kernel<T, V><<<(unsigned)BT, 128, 0, st>>>((const T*)x, ang, (const T*)dy, (T*)out, dang, H, D, aH)));
        else SSD_LAUNCH(ssd::prof::K_TC_AUX, st, (rope_op_bwd_kernel<T, 2><<<(unsigned)BT, 128, 0, st>>>((const T*)x, ang, (const T*)dy, (T*)out, dang, H, D, aH)));
    }
    CUDA_LAUNCH_CHECK("rope");
    return 0;
}

template <class T>
int trapezoid_impl(bool backward, size_t M, int H, const void* dt_raw, const void* lam_raw, const float* dt_bias,
                   const float* A_log, const void* const* g, void* const* out, float* d_dt_bias, float* d_A_log,
                   float* part_ws, cudaStream_t st) {
    using namespace ssd::ew;
    if (!backward) {
        const size_t total = M * (size_t)H;
        SSD_LAUNCH(ssd::prof::K_TC_AUX, st, trapezoid_fwd_kernel<T><<<(unsigned)((total + 255) / 256), 256, 0, st>>>((const T*)dt_raw, (const T*)lam_raw, dt_bias, A_log, (T*)out[0], (T*)out[1], (T*)out[2], (T*)out[3], total, H));
    } else {
        const size_t nblk = (M + TRAP_ROWS - 1) / TRAP_ROWS;
        float* pb = part_ws;
        float* pa = part_ws + nblk * H;
        SSD_LAUNCH(ssd::prof::K_TC_AUX, st, trapezoid_bwd_kernel<T><<<(unsigned)nblk, 256, 0, st>>>((const T*)dt_raw, (const T*)lam_raw, dt_bias, A_log, (const T*)g[0], (const T*)g[1], (const T*)g[2], (const T*)g[3], (T*)out[0], (T*)out[1], pb, pa, M, H));
        SSD_LAUNCH(ssd::prof::K_REDUCE, st, ssd::tc::reduce_rows_kernel<<<dim3(H, 2), 256, 0, st>>>(pb, d_dt_bias, (int)nblk, H, pa, d_A_log));
    }
    CUDA_LAUNCH_CHECK("trapezoid");
    return 0;
}

template <class T>
int rmsnorm_impl(bool backward, size_t M, int D, float eps, const void* x, const float* w, const void* z, const void* dout,
                 void* out, void* dz, float* rstd, float* dw, float* part_ws, cudaStream_t st, const float* ysq = nullptr,
                 int ysq_heads = 0) {
    using namespace ssd::ew;
    constexpr int V = VecOf<T>::N;
    const bool vec = D % V == 0;
    const unsigned blocks = (unsigned)((M + 7) / 8);
    if (!backward) {
        if (vec) SSD_LAUNCH(ssd::prof::K_TC_AUX, st, (rmsnorm_fwd_kernel<T, V><<<blocks, 256, 0, st>>>((const T*)x, w, (const T*)z, (T*)out, rstd, M, D, eps, ysq, ysq_heads)));
        else SSD_LAUNCH(ssd::prof::K_TC_AUX, st, (rmsnorm_fwd_kernel<T, 1><<<blocks, 256, 0, st>>>((const T*)x, w, (const T*)z, (T*)out, rstd, M, D, eps, ysq, ysq_heads)));
    } else {
        if (vec) SSD_LAUNCH(ssd::prof::K_TC_AUX, st, (rmsnorm_bwd_kernel<T, V><<<blocks, 256, 0, st>>>((const T*)x, w, (const T*)z, (const T*)dout, rstd, (T*)out, (T*)dz, M, D)));
        else SSD_LAUNCH(ssd::prof::K_TC_AUX, st, (rmsnorm_bwd_kernel<T, 1><<<blocks, 256, 0, st>>>((const T*)x, w, (const T*)z, (const T*)dout, rstd, (T*)out, (T*)dz, M, D)));
        const unsigned chunks = (unsigned)((M + RMS_ROWS - 1) / RMS_ROWS);
        if (vec) SSD_LAUNCH(ssd::prof::K_TC_AUX, st, (rmsnorm_dw_kernel<T, V><<<dim3((D + 32 * V - 1) / (32 * V), chunks), 256, 0, st>>>((const T*)x, (const T*)z, (const T*)dout, rstd, part_ws, M, D)));
        else SSD_LAUNCH(ssd::prof::K_TC_AUX, st, (rmsnorm_dw_kernel<T, 1><<<dim3((D + 31) / 32, chunks), 256, 0, st>>>((const T*)x, (const T*)z, (const T*)dout, rstd, part_ws, M, D)));
        SSD_LAUNCH(ssd::prof::K_REDUCE, st, ssd::tc::reduce_rows_kernel<<<D, 256, 0, st>>>(part_ws, dw, (int)chunks, D));
    }
    CUDA_LAUNCH_CHECK("rmsnorm");
    return 0;
}
}  // namespace


extern "C" {

int ssd_b200_abi_version(void) { return SSD_B200_ABI_VERSION; }

long long ssd_b200_launch_count(void) { return ssd::prof::g_launches.load(); }

int ssd_b200_profile_enable(int on) {
    ssd::prof::g_enabled = on != 0;
    return 0;
}

int ssd_b200_profile_kernels(void) { return ssd::prof::K_COUNT; }

const char* ssd_b200_profile_kernel_name(int idx) {
    return (idx >= 0 && idx < ssd::prof::K_COUNT) ? ssd::prof::kNames[idx] : "";
}

int ssd_b200_profile_read(float* ms, long long* launches, int n) {
    if (!ms || !launches || n < ssd::prof::K_COUNT) return fail(SSD_B200_EINVAL, "profile_read needs %d slots", ssd::prof::K_COUNT);
    for (int i = 0; i < n; ++i) { ms[i] = 0.f; launches[i] = 0; }
    int rc = 0;
    for (auto& r : ssd::prof::g_recs) {
        float t = 0.f;
        if (cudaEventSynchronize(r.b) != cudaSuccess || cudaEventElapsedTime(&t, r.a, r.b) != cudaSuccess) rc = SSD_B200_ECUDA;
        ms[r.k] += t;
        launches[r.k] += 1;
        cudaEventDestroy(r.a);
        cudaEventDestroy(r.b);
    }
    ssd::prof::g_recs.clear();
    if (rc) return fail(rc, "profile_read: event query failed");
    return 0;
}

const char* ssd_b200_last_error(void) { return g_err; }

int ssd_b200_resolve_path(const ssd_b200_shape* shape) {
    if (int rc = check_shape(shape)) return rc;
    return resolve_path(*shape);
}

size_t ssd_b200_workspace_bytes(const ssd_b200_shape* shape, int pass) {
    if (check_shape(shape)) return 0;
    if (pass != SSD_B200_PASS_FWD && pass != SSD_B200_PASS_BWD) return 0;
    int path = resolve_path(*shape);
    if (path < 0) return 0;
    ssd::Dims d = dims_of(*shape);
    if (path == SSD_B200_PATH_TC) return ssd::tc::workspace_bytes(d, pass);
    return simt_ws(d, pass).total;
}

size_t ssd_b200_states_bytes(const ssd_b200_shape* shape) {
    if (check_shape(shape)) return 0;
    if (resolve_path(*shape) != SSD_B200_PATH_TC) return 0;
    return ssd::tc::states_bytes(dims_of(*shape));
}

int ssd_b200_fwd(const ssd_b200_fwd_args* a, void* stream) {
    if (!a) return fail(SSD_B200_EINVAL, "args is null");
    if (int rc = check_shape(&a->shape)) return rc;
    const int form = check_forms(a->a, a->dt, a->A_head, a->D, a->skip);
    if (form < 0) return form;
    const bool states_only = (a->flags & SSD_B200_FWD_STATES_ONLY) != 0;
    if (!a->x || !a->B || !a->C || !a->a_cumsum || (!a->y && !states_only)) return fail(SSD_B200_EINVAL, "null tensor pointer");
    if (states_only && !a->final_state) return fail(SSD_B200_EINVAL, "STATES_ONLY needs final_state");
    int path = resolve_path(a->shape);
    if (path < 0) return path;
    if (!a->workspace || ((uintptr_t)a->workspace & 255)) return fail(SSD_B200_EWORKSPACE, "workspace null or not 256-byte aligned");
    cudaStream_t st = (cudaStream_t)stream;
    if (a->states && path != SSD_B200_PATH_TC) return fail(SSD_B200_EINVAL, "`states` is only used by the tensor-core path");
    if (a->ysq && path != SSD_B200_PATH_TC) return fail(SSD_B200_EINVAL, "`ysq` is only written by the tensor-core path");
    if (form == 3 && path != SSD_B200_PATH_TC) return fail(SSD_B200_EUNSUPPORTED, "the scaled operator form needs the tensor-core path");
    if (path == SSD_B200_PATH_TC) return ssd::tc::forward(a, dims_of(a->shape), st, g_err, sizeof(g_err));
    return a->shape.dtype == SSD_B200_BF16 ? simt_fwd<__nv_bfloat16>(a, st) : simt_fwd<float>(a, st);
}

int ssd_b200_bwd(const ssd_b200_bwd_args* a, void* stream) {
    if (!a) return fail(SSD_B200_EINVAL, "args is null");
    if (int rc = check_shape(&a->shape)) return rc;
    int form = 0;
    if (!(a->flags & SSD_B200_BWD_DINIT_ONLY)) {
        form = check_forms(a->a, a->dt, a->A_head, a->D, a->skip);
        if (form < 0) return form;
    }
    const bool dinit_only = (a->flags & SSD_B200_BWD_DINIT_ONLY) != 0;
    if (dinit_only) {
        if (!a->C || !a->dy || !a->a_cumsum || !a->dinit) return fail(SSD_B200_EINVAL, "DINIT_ONLY needs C, dy, a_cumsum and dinit");
    } else {
        if (!a->x || !a->B || !a->C || !a->dy || !a->a_cumsum || !a->dx || !a->dB || !a->dC)
            return fail(SSD_B200_EINVAL, "null tensor pointer");
        if (form == 2 && (!a->ddt || !a->dA_head || (a->D && !a->dD))) return fail(SSD_B200_EINVAL, "Mamba-2 form needs ddt, dA_head (and dD)");
        if (form == 3 && (!a->ddt || (a->skip && !a->dskip))) return fail(SSD_B200_EINVAL, "scaled operator form needs ddt (and dskip)");
        if (a->a && !a->cumsum_is_input && !a->da) return fail(SSD_B200_EINVAL, "operator form needs da");
    }
    int path = resolve_path(a->shape);
    if (path < 0) return path;
    if (!a->workspace || ((uintptr_t)a->workspace & 255)) return fail(SSD_B200_EWORKSPACE, "workspace null or not 256-byte aligned");
    cudaStream_t st = (cudaStream_t)stream;
    if (a->states && path != SSD_B200_PATH_TC) return fail(SSD_B200_EINVAL, "`states` is only used by the tensor-core path");
    if (form == 3 && path != SSD_B200_PATH_TC) return fail(SSD_B200_EUNSUPPORTED, "the scaled operator form needs the tensor-core path");
    if (path == SSD_B200_PATH_TC) return ssd::tc::backward(a, dims_of(a->shape), st, g_err, sizeof(g_err));
    return a->shape.dtype == SSD_B200_BF16 ? simt_bwd<__nv_bfloat16>(a, st) : simt_bwd<float>(a, st);
}

// ------------------------------------------------------------------------------------------
// Forward for callers that cannot hand over a workspace.
//
// Some hosts only ever see the device pointers of their inputs and outputs: a plugin running under
// a framework that owns the whole device-memory pool and gives plugins no allocator, or a process
// started with a fixed device-memory reservation in which cudaMalloc after start-up is not allowed.
// Such a caller has nowhere to get the scratch buffer ssd_b200_fwd asks for.  For them the library
// carries its own scratch: one fixed array in device memory, part of the loaded module.
//
// The array below exists once per GPU that loads this library and stays until the process exits.
// In host code its name is only a handle, not a device address; the address comes from
// cudaGetSymbolAddress, which is asked on EVERY call: the answer belongs to the CUDA context that is
// current on the calling thread, so a value remembered from an earlier call could be stale after a
// device reset or belong to another context on the same GPU.  The lookup is a host-side table read
// and allocates nothing; the very first one on a device loads the library's device code there.
// ------------------------------------------------------------------------------------------
#define SSD_B200_STATIC_SCRATCH_BYTES (64u << 20)
static __device__ __align__(256) unsigned char g_static_scratch[SSD_B200_STATIC_SCRATCH_BYTES];

namespace {
int static_scratch_on_current_device(void** out) {
    void* p = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&p, g_static_scratch);
    if (e != cudaSuccess || !p)
        return fail(SSD_B200_ECUDA, "cudaGetSymbolAddress(static scratch): %s", cudaGetErrorString(e));
    *out = p;
    return 0;
}
}  // namespace

int ssd_b200_fwd_static_scratch(const ssd_b200_fwd_args* a, void* stream) {
    if (!a) return fail(SSD_B200_EINVAL, "args is null");
    if (int rc = check_shape(&a->shape)) return rc;
    int path = resolve_path(a->shape);
    if (path < 0) return path;
    const size_t need = ssd_b200_workspace_bytes(&a->shape, SSD_B200_PASS_FWD);
    if (need > (size_t)SSD_B200_STATIC_SCRATCH_BYTES)
        return fail(SSD_B200_EWORKSPACE,
                    "this shape needs %zu bytes of scratch but the built-in array holds %u; use ssd_b200_fwd with a "
                    "caller workspace", need, (unsigned)SSD_B200_STATIC_SCRATCH_BYTES);
    void* scratch = nullptr;
    if (int rc = static_scratch_on_current_device(&scratch)) return rc;
    ssd_b200_fwd_args b = *a;
    b.workspace = scratch;
    b.workspace_bytes = (size_t)SSD_B200_STATIC_SCRATCH_BYTES;
    return ssd_b200_fwd(&b, stream);
}

size_t ssd_b200_static_scratch_bytes(void) { return (size_t)SSD_B200_STATIC_SCRATCH_BYTES; }

int ssd_b200_device_status(const ssd_b200_shape* shape, const void* workspace, void* stream) {
    if (int rc = check_shape(shape)) return rc;
    if (!workspace) {  // the caller of ssd_b200_fwd_static_scratch never sees the scratch address
        void* scratch = nullptr;
        if (int rc = static_scratch_on_current_device(&scratch)) return rc;
        workspace = scratch;
    }
    int path = resolve_path(*shape);
    if (path < 0) return path;
    if (path != SSD_B200_PATH_TC) return 0;  // only the tensor-core kernels have bounded waits to report
    int status = 0;
    cudaStream_t st = (cudaStream_t)stream;
    cudaError_t e = cudaMemcpyAsync(&status, workspace, sizeof(int), cudaMemcpyDeviceToHost, st);
    if (e == cudaSuccess) e = cudaStreamSynchronize(st);
    if (e != cudaSuccess) return fail(SSD_B200_ECUDA, "device_status: %s", cudaGetErrorString(e));
    if (status != 0) return fail(SSD_B200_EDEVICE, "a kernel gave up on a bounded wait (status %d); results are invalid", status);
    return 0;
}

int ssd_b200_selftest_bounded_wait(void* workspace, int32_t polls, void* stream) {
    if (!workspace || ((uintptr_t)workspace & 3)) return fail(SSD_B200_EWORKSPACE, "workspace null or misaligned");
    if (polls <= 0 || polls > (1 << 20)) return fail(SSD_B200_EINVAL, "polls must be in [1, 2^20]");
    cudaStream_t st = (cudaStream_t)stream;
    if (cudaMemsetAsync(workspace, 0, 4, st) != cudaSuccess) return fail(SSD_B200_ECUDA, "memset failed");
    SSD_LAUNCH(ssd::prof::K_TC_AUX, st, ssd::tc::bounded_wait_selftest_kernel<<<1, 32, 0, st>>>((int*)workspace, polls));
    CUDA_LAUNCH_CHECK("bounded_wait_selftest");
    return 0;
}

int ssd_b200_m3_prologue_fwd(const ssd_b200_shape* shape, const void* x, const float* dt, const float* lam,
                             const float* A_head, const void* B, const void* C, const void* raw_angles, int32_t angles_dtype,
                             void* xw, float* dA, void* Br, void* Cr, float* sdot, float* cum, float* segsum_ws, const float* D,
                             float* w_out, float* skip_out, void* stream) {
    if (int rc = check_shape(shape)) return rc;
    if (!dt || !lam || !A_head || !B || !C || !raw_angles || !dA || !Br || !Cr || !sdot || !cum || !segsum_ws)
        return fail(SSD_B200_EINVAL, "null pointer");
    if (xw ? !x : (!w_out || !skip_out)) return fail(SSD_B200_EINVAL, "give x and xw, or w_out and skip_out");
    if (angles_dtype != SSD_B200_F32 && angles_dtype != shape->dtype) return fail(SSD_B200_EINVAL, "raw_angles must be fp32 or in the storage dtype");
    if (shape->dstate % 2) return fail(SSD_B200_EINVAL, "d_state must be even for the pairwise rotation");
    ssd::Dims d = dims_of(*shape);
    if (d.T > 65535 || d.b > 65535) return fail(SSD_B200_EUNSUPPORTED, "grid dimension too large");
    cudaStream_t st = (cudaStream_t)stream;
    const bool af = angles_dtype == SSD_B200_F32;
    return shape->dtype == SSD_B200_BF16
               ? m3_fwd_impl<__nv_bfloat16>(d, x, dt, lam, A_head, B, C, raw_angles, af, xw, dA, Br, Cr, sdot, cum, segsum_ws, D, w_out, skip_out, st)
               : m3_fwd_impl<float>(d, x, dt, lam, A_head, B, C, raw_angles, af, xw, dA, Br, Cr, sdot, cum, segsum_ws, D, w_out, skip_out, st);
}

int ssd_b200_m3_skip_fwd(const ssd_b200_shape* shape, const void* y_scan, const void* x, const float* D, const float* dt,
                         const float* lam, const float* sdot, void* y, void* stream) {
    if (int rc = check_shape(shape)) return rc;
    if (!y_scan || !x || !dt || !lam || !sdot || !y) return fail(SSD_B200_EINVAL, "null pointer");
    ssd::Dims d = dims_of(*shape);
    cudaStream_t st = (cudaStream_t)stream;
    return shape->dtype == SSD_B200_BF16 ? m3_skip_impl<__nv_bfloat16>(d, y_scan, x, D, dt, lam, sdot, y, st)
                                         : m3_skip_impl<float>(d, y_scan, x, D, dt, lam, sdot, y, st);
}

size_t ssd_b200_m3_chain_ws_floats(const ssd_b200_shape* shape) {
    if (!shape || shape->batch <= 0 || shape->seqlen <= 0 || shape->nheads <= 0) return 0;
    const size_t M = (size_t)shape->batch * shape->seqlen;
    return 2 * ((M + ssd::m3::CHAIN_ROWS - 1) / ssd::m3::CHAIN_ROWS) * (size_t)shape->nheads;
}

int ssd_b200_m3_chain_bwd(const ssd_b200_shape* shape, const float* dw, const float* dyx, const float* sdot, const float* dt,
                          const float* lam, const float* da, const float* A_head, float* dlam, float* ddt, float* dA_head,
                          float* dD, float* ws, void* stream) {
    if (int rc = check_shape(shape)) return rc;
    if (!dw || !dyx || !sdot || !dt || !lam || !da || !A_head || !dlam || !ddt || !dA_head || !ws)
        return fail(SSD_B200_EINVAL, "null pointer");
    ssd::Dims d = dims_of(*shape);
    cudaStream_t st = (cudaStream_t)stream;
    const size_t M = (size_t)d.b * d.T, nblk = (M + ssd::m3::CHAIN_ROWS - 1) / ssd::m3::CHAIN_ROWS;
    float* pA = ws;
    float* pD = ws + nblk * d.h;
    SSD_LAUNCH(ssd::prof::K_TC_AUX, st, ssd::m3::chain_bwd_kernel<<<(unsigned)nblk, 256, 0, st>>>(dw, dyx, sdot, dt, lam, da, A_head, dlam, ddt, pA, pD, M, d.T, d.h, d.g));
    SSD_LAUNCH(ssd::prof::K_REDUCE, st, ssd::tc::reduce_rows_kernel<<<dim3(d.h, dD ? 2 : 1), 256, 0, st>>>(pA, dA_head, (int)nblk, d.h, pD, dD));
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return fail(SSD_B200_ECUDA, cudaGetErrorString(e));
    return SSD_B200_OK;
}

int ssd_b200_m3_prologue_bwd(const ssd_b200_shape* shape, const void* x, const void* dy, const float* dt, const float* lam,
                             const float* D, const void* B, const void* C, const float* cum, const float* sdot,
                             const void* dxw, const void* dBr, const void* dCr, void* dx, float* dw, float* dyx, void* dB,
                             void* dC, void* d_raw_angles, int32_t angles_dtype, float* dcum_ws, float* segsum_ws,
                             void* stream) {
    if (int rc = check_shape(shape)) return rc;
    if (!dt || !lam || !B || !C || !cum || !sdot || !dBr || !dCr || !dw || !dyx || !dB || !dC || !d_raw_angles || !dcum_ws ||
        !segsum_ws)
        return fail(SSD_B200_EINVAL, "null pointer");
    if (dxw && (!x || !dy || !dx)) return fail(SSD_B200_EINVAL, "with dxw given, x, dy and dx are needed");
    if (angles_dtype != SSD_B200_F32 && angles_dtype != shape->dtype) return fail(SSD_B200_EINVAL, "d_raw_angles must be fp32 or in the storage dtype");
    if (shape->dstate % 2) return fail(SSD_B200_EINVAL, "d_state must be even for the pairwise rotation");
    ssd::Dims d = dims_of(*shape);
    if (d.T > 65535 || d.b > 65535) return fail(SSD_B200_EUNSUPPORTED, "grid dimension too large");
    cudaStream_t st = (cudaStream_t)stream;
    const bool af = angles_dtype == SSD_B200_F32;
    return shape->dtype == SSD_B200_BF16
               ? m3_bwd_impl<__nv_bfloat16>(d, x, dy, dt, lam, D, B, C, cum, sdot, dxw, dBr, dCr, dx, dw, dyx, dB, dC, d_raw_angles, af, dcum_ws, segsum_ws, st)
               : m3_bwd_impl<float>(d, x, dy, dt, lam, D, B, C, cum, sdot, dxw, dBr, dCr, dx, dw, dyx, dB, dC, d_raw_angles, af, dcum_ws, segsum_ws, st);
}

int ssd_b200_rope_fwd(int32_t dtype, int64_t B, int64_t T, int64_t H, int64_t D, int32_t broadcast_h, const void* x,
                      const float* angles, void* y, void* stream) {
    if (!x || !angles || !y) return fail(SSD_B200_EINVAL, "null pointer");
    if (B <= 0 || T <= 0 || H <= 0 || D <= 0 || D % 2 || B * T > 2147483647LL) return fail(SSD_B200_EINVAL, "bad rope dimensions");
    const int aH = broadcast_h ? 1 : (int)H;
    cudaStream_t st = (cudaStream_t)stream;
    if (dtype == SSD_B200_BF16) return rope_op_impl<__nv_bfloat16>(false, B * T, (int)H, (int)D, aH, x, angles, nullptr, y, nullptr, st);
    if (dtype == SSD_B200_F32) return rope_op_impl<float>(false, B * T, (int)H, (int)D, aH, x, angles, nullptr, y, nullptr, st);
    return fail(SSD_B200_EUNSUPPORTED, "dtype %d", dtype);
}

int ssd_b200_rope_bwd(int32_t dtype, int64_t B, int64_t T, int64_t H, int64_t D, int32_t broadcast_h, const void* x,
                      const float* angles, const void* dy, void* dx, float* dangles, void* stream) {
    if (!x || !angles || !dy || !dx || !dangles) return fail(SSD_B200_EINVAL, "null pointer");
    if (B <= 0 || T <= 0 || H <= 0 || D <= 0 || D % 2 || B * T > 2147483647LL) return fail(SSD_B200_EINVAL, "bad rope dimensions");
    const int aH = broadcast_h ? 1 : (int)H;
    cudaStream_t st = (cudaStream_t)stream;
    if (dtype == SSD_B200_BF16) return rope_op_impl<__nv_bfloat16>(true, B * T, (int)H, (int)D, aH, x, angles, dy, dx, dangles, st);
    if (dtype == SSD_B200_F32) return rope_op_impl<float>(true, B * T, (int)H, (int)D, aH, x, angles, dy, dx, dangles, st);
    return fail(SSD_B200_EUNSUPPORTED, "dtype %d", dtype);
}

size_t ssd_b200_trapezoid_ws_floats(int64_t rows, int64_t H) {
    if (rows <= 0 || H <= 0) return 0;
    return (size_t)2 * (size_t)((rows + ssd::ew::TRAP_ROWS - 1) / ssd::ew::TRAP_ROWS) * (size_t)H;
}

int ssd_b200_trapezoid_fwd(int32_t dtype, int64_t rows, int64_t H, const void* dt_raw, const void* lam_raw,
                           const float* dt_bias, const float* A_log, void* dt, void* dA, void* beta, void* gamma,
                           void* stream) {
    if (!dt_raw || !lam_raw || !dt_bias || !A_log || !dt || !dA || !beta || !gamma) return fail(SSD_B200_EINVAL, "null pointer");
    if (rows <= 0 || H <= 0 || H > 2147483647LL) return fail(SSD_B200_EINVAL, "bad trapezoid dimensions");
    void* out[4] = {dt, dA, beta, gamma};
    cudaStream_t st = (cudaStream_t)stream;
    if (dtype == SSD_B200_BF16) return trapezoid_impl<__nv_bfloat16>(false, (size_t)rows, (int)H, dt_raw, lam_raw, dt_bias, A_log, nullptr, out, nullptr, nullptr, nullptr, st);
    if (dtype == SSD_B200_F32) return trapezoid_impl<float>(false, (size_t)rows, (int)H, dt_raw, lam_raw, dt_bias, A_log, nullptr, out, nullptr, nullptr, nullptr, st);
    return fail(SSD_B200_EUNSUPPORTED, "dtype %d", dtype);
}

int ssd_b200_trapezoid_bwd(int32_t dtype, int64_t rows, int64_t H, const void* dt_raw, const void* lam_raw,
                           const float* dt_bias, const float* A_log, const void* g_dt, const void* g_dA, const void* g_beta,
                           const void* g_gamma, void* d_dt_raw, void* d_lam_raw, float* d_dt_bias, float* d_A_log,
                           float* ws, void* stream) {
    if (!dt_raw || !lam_raw || !dt_bias || !A_log || !g_dt || !g_dA || !g_beta || !g_gamma || !d_dt_raw || !d_lam_raw ||
        !d_dt_bias || !d_A_log || !ws)
        return fail(SSD_B200_EINVAL, "null pointer");
    if (rows <= 0 || H <= 0 || H > 65535) return fail(SSD_B200_EINVAL, "bad trapezoid dimensions");
    const void* g[4] = {g_dt, g_dA, g_beta, g_gamma};
    void* out[2] = {d_dt_raw, d_lam_raw};
    cudaStream_t st = (cudaStream_t)stream;
    if (dtype == SSD_B200_BF16) return trapezoid_impl<__nv_bfloat16>(true, (size_t)rows, (int)H, dt_raw, lam_raw, dt_bias, A_log, g, out, d_dt_bias, d_A_log, ws, st);
    if (dtype == SSD_B200_F32) return trapezoid_impl<float>(true, (size_t)rows, (int)H, dt_raw, lam_raw, dt_bias, A_log, g, out, d_dt_bias, d_A_log, ws, st);
    return fail(SSD_B200_EUNSUPPORTED, "dtype %d", dtype);
}

size_t ssd_b200_rmsnorm_ws_floats(int64_t rows, int64_t D) {
    if (rows <= 0 || D <= 0) return 0;
    return (size_t)((rows + ssd::ew::RMS_ROWS - 1) / ssd::ew::RMS_ROWS) * (size_t)D;
}

int ssd_b200_rmsnorm_fwd(int32_t dtype, int64_t rows, int64_t D, float eps, const void* x, const float* weight,
                         const void* z, void* out, float* rstd, void* stream) {
    if (!x || !weight || !out || !rstd) return fail(SSD_B200_EINVAL, "null pointer");
    if (rows <= 0 || D <= 0 || D > 2147483647LL || (rows + 7) / 8 > 2147483647LL) return fail(SSD_B200_EINVAL, "bad rmsnorm dimensions");
    cudaStream_t st = (cudaStream_t)stream;
    if (dtype == SSD_B200_BF16) return rmsnorm_impl<__nv_bfloat16>(false, (size_t)rows, (int)D, eps, x, weight, z, nullptr, out, nullptr, rstd, nullptr, nullptr, st);
    if (dtype == SSD_B200_F32) return rmsnorm_impl<float>(false, (size_t)rows, (int)D, eps, x, weight, z, nullptr, out, nullptr, rstd, nullptr, nullptr, st);
    return fail(SSD_B200_EUNSUPPORTED, "dtype %d", dtype);
}

int ssd_b200_rmsnorm_fwd_presummed(int32_t dtype, int64_t rows, int64_t D, float eps, const void* x, const float* weight,
                                   const void* z, const float* ysq, int64_t nheads, void* out, float* rstd, void* stream) {
    if (!x || !weight || !out || !rstd || !ysq) return fail(SSD_B200_EINVAL, "null pointer");
    if (rows <= 0 || D <= 0 || D > 2147483647LL || (rows + 7) / 8 > 2147483647LL || nheads <= 0 || nheads > 32767 || rows % 128)
        return fail(SSD_B200_EINVAL, "bad rmsnorm dimensions (rows must be a multiple of 128)");
    cudaStream_t st = (cudaStream_t)stream;
    if (dtype == SSD_B200_BF16) return rmsnorm_impl<__nv_bfloat16>(false, (size_t)rows, (int)D, eps, x, weight, z, nullptr, out, nullptr, rstd, nullptr, nullptr, st, ysq, (int)nheads);
    if (dtype == SSD_B200_F32) return rmsnorm_impl<float>(false, (size_t)rows, (int)D, eps, x, weight, z, nullptr, out, nullptr, rstd, nullptr, nullptr, st, ysq, (int)nheads);
    return fail(SSD_B200_EUNSUPPORTED, "dtype %d", dtype);
}

int ssd_b200_rmsnorm_bwd(int32_t dtype, int64_t rows, int64_t D, const void* x, const float* weight, const void* z,
                         const void* dout, const float* rstd, void* dx, void* dz, float* dweight, float* ws, void* stream) {
    if (!x || !weight || !dout || !rstd || !dx || !dweight || !ws || (z && !dz)) return fail(SSD_B200_EINVAL, "null pointer");
    if (rows <= 0 || D <= 0 || D > 65535 * 32LL || (rows + 7) / 8 > 2147483647LL || (rows + ssd::ew::RMS_ROWS - 1) / ssd::ew::RMS_ROWS > 65535)
        return fail(SSD_B200_EINVAL, "bad rmsnorm dimensions");
    cudaStream_t st = (cudaStream_t)stream;
    if (dtype == SSD_B200_BF16) return rmsnorm_impl<__nv_bfloat16>(true, (size_t)rows, (int)D, 0.f, x, weight, z, dout, dx, dz, const_cast<float*>(rstd), dweight, ws, st);
    if (dtype == SSD_B200_F32) return rmsnorm_impl<float>(true, (size_t)rows, (int)D, 0.f, x, weight, z, dout, dx, dz, const_cast<float*>(rstd), dweight, ws, st);
    return fail(SSD_B200_EUNSUPPORTED, "dtype %d", dtype);
}

int ssd_b200_materialize_cache(const ssd_b200_shape* shape, const float* a_cumsum, void* L, void* decay_chunk,
                               int32_t dtype, void* stream) {
    if (int rc = check_shape(shape)) return rc;
    if (!a_cumsum) return fail(SSD_B200_EINVAL, "a_cumsum is null");
    ssd::Dims d = dims_of(*shape);
    cudaStream_t st = (cudaStream_t)stream;
    const size_t chunks = (size_t)d.b * d.h * d.c;
    if (chunks > 2147483647u) return fail(SSD_B200_EUNSUPPORTED, "too many chunks");
    if (L) {
        if (dtype == SSD_B200_BF16)
            SSD_LAUNCH(ssd::prof::K_CACHE_L, st, ssd::simt::cache_L_kernel<<<(unsigned)chunks, 256, 0, st>>>(a_cumsum, (__nv_bfloat16*)L, chunks, d.l));
        else
            SSD_LAUNCH(ssd::prof::K_CACHE_L, st, ssd::simt::cache_L_kernel<<<(unsigned)chunks, 256, 0, st>>>(a_cumsum, (float*)L, chunks, d.l));
        CUDA_LAUNCH_CHECK("cache_L");
    }
    if (decay_chunk) {
        if (d.c + 1 > 65535) return fail(SSD_B200_EUNSUPPORTED, "too many chunks for decay_chunk");
        dim3 g((unsigned)(d.b * d.h), d.c + 1);
        if (dtype == SSD_B200_BF16)
            SSD_LAUNCH(ssd::prof::K_CACHE_DC, st, ssd::simt::cache_decay_chunk_kernel<<<g, 128, 0, st>>>(a_cumsum, (__nv_bfloat16*)decay_chunk, d.c, d.l));
        else
            SSD_LAUNCH(ssd::prof::K_CACHE_DC, st, ssd::simt::cache_decay_chunk_kernel<<<g, 128, 0, st>>>(a_cumsum, (float*)decay_chunk, d.c, d.l));
        CUDA_LAUNCH_CHECK("cache_decay_chunk");
    }
    return 0;
}

// CUDA IPC of a device buffer between the processes of one node.  The importing side opens the handle with ITS OWN
// device current and cudaIpcMemLazyEnablePeerAccess, which is what makes the mapping usable by kernels of that device
// when the memory lives on another GPU.
int ssd_b200_ipc_export(const void* ptr, unsigned char* handle64, int64_t* offset) {
    if (!ptr || !handle64 || !offset) return fail(SSD_B200_EINVAL, "null pointer");
    typedef CUresult (*RangeFn)(CUdeviceptr*, size_t*, CUdeviceptr);
    static RangeFn range = [] {
        void* f = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuMemGetAddressRange", &f, cudaEnableDefault, &q) != cudaSuccess) f = nullptr;
        return (RangeFn)f;
    }();
    if (!range) return fail(SSD_B200_ECUDA, "cuMemGetAddressRange is not available");
    CUdeviceptr base = 0;
    size_t size = 0;
    if (range(&base, &size, (CUdeviceptr)ptr) != CUDA_SUCCESS) return fail(SSD_B200_ECUDA, "cuMemGetAddressRange failed");
    cudaIpcMemHandle_t h;
    cudaError_t e = cudaIpcGetMemHandle(&h, (void*)base);
    if (e != cudaSuccess) return fail(SSD_B200_ECUDA, "cudaIpcGetMemHandle: %s", cudaGetErrorString(e));
    static_assert(sizeof(h) == 64, "IPC handle size");
    memcpy(handle64, &h, 64);
    *offset = (int64_t)((CUdeviceptr)ptr - base);
    return 0;
}

int ssd_b200_ipc_import(const unsigned char* handle64, void** base_out) {
    if (!handle64 || !base_out) return fail(SSD_B200_EINVAL, "null pointer");
    cudaIpcMemHandle_t h;
    memcpy(&h, handle64, 64);
    void* p = nullptr;
    cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return fail(SSD_B200_ECUDA, "cudaIpcOpenMemHandle: %s", cudaGetErrorString(e));
    }
    unsigned int probe = 0;  // a copy through the runtime fails with an error code (not a fault) if the mapping is unusable
    e = cudaMemcpy(&probe, p, sizeof(probe), cudaMemcpyDeviceToHost);
    if (e != cudaSuccess) {
        cudaGetLastError();
        cudaIpcCloseMemHandle(p);
        return fail(SSD_B200_ECUDA, "imported memory is not readable from this device: %s", cudaGetErrorString(e));
    }
    *base_out = p;
    return 0;
}

int ssd_b200_ipc_close(void* base) {
    if (!base) return 0;
    cudaError_t e = cudaIpcCloseMemHandle(base);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return fail(SSD_B200_ECUDA, "cudaIpcCloseMemHandle: %s", cudaGetErrorString(e));
    }
    return 0;
}

int ssd_b200_enable_peer_access(int32_t peer_device) {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess) return fail(SSD_B200_ECUDA, "cudaGetDevice failed");
    if (peer_device == dev) return 0;
    int can = 0;
    cudaError_t e = cudaDeviceCanAccessPeer(&can, dev, peer_device);
    if (e != cudaSuccess || !can) return fail(SSD_B200_EUNSUPPORTED, "device %d cannot access device %d as a peer", dev, peer_device);
    e = cudaDeviceEnablePeerAccess(peer_device, 0);
    if (e == cudaErrorPeerAccessAlreadyEnabled) {
        cudaGetLastError();  // clear the sticky-less error state
        return 0;
    }
    if (e != cudaSuccess) return fail(SSD_B200_ECUDA, "cudaDeviceEnablePeerAccess(%d): %s", peer_device, cudaGetErrorString(e));
    return 0;
}

int ssd_b200_exchange_push(const float* src, int64_t n, float* const* peer_bufs, int64_t nranks, int64_t dst_offset,
                           void* stream) {
    if (!src || !peer_bufs) return fail(SSD_B200_EINVAL, "null pointer");
    if (n <= 0 || n % 4 || nranks <= 0 || nranks > 32 || dst_offset < 0 || dst_offset % 4 || ((uintptr_t)src & 15))
        return fail(SSD_B200_EINVAL, "exchange_push: sizes and offsets must be positive multiples of 4 floats, src 16-byte aligned");
    const size_t n4 = (size_t)n / 4;
    cudaStream_t st = (cudaStream_t)stream;
    SSD_LAUNCH(ssd::prof::K_EXCHANGE, st, ssd::simt::exchange_push_kernel<<<(unsigned)((n4 + 255) / 256), 256, 0, st>>>(
        (const float4*)src, n4, peer_bufs, (int)nranks, (size_t)dst_offset));
    CUDA_LAUNCH_CHECK("exchange_push");
    return 0;
}

int ssd_b200_exchange_arrive(unsigned int* const* peer_flags, int64_t rank, int64_t nranks, uint32_t epoch, int32_t* status,
                             uint32_t max_polls, void* stream) {
    if (!peer_flags || !status) return fail(SSD_B200_EINVAL, "null pointer");
    if (nranks <= 0 || nranks > 32 || rank < 0 || rank >= nranks || max_polls == 0) return fail(SSD_B200_EINVAL, "bad exchange_arrive arguments");
    cudaStream_t st = (cudaStream_t)stream;
    SSD_LAUNCH(ssd::prof::K_EXCHANGE, st, ssd::simt::exchange_arrive_kernel<<<1, 32, 0, st>>>(peer_flags, (int)rank, (int)nranks, epoch, status, max_polls));
    CUDA_LAUNCH_CHECK("exchange_arrive");
    return 0;
}

int ssd_b200_state_prefix_all(const float* pieces, const float* logp, const float* edge, float* out, float* total,
                              float* total_logp, int64_t nranks, int64_t rank, int64_t segments, int64_t batch,
                              int64_t nheads, int64_t state_elems, int64_t rank_stride, int64_t logp_stride, int32_t reverse,
                              const float* outer, const float* outer_logp, int64_t outer_n, int64_t outer_rank,
                              int64_t outer_stride, int64_t outer_logp_stride, void* stream) {
    if (!pieces || !logp || (!out && !total)) return fail(SSD_B200_EINVAL, "null pointer");
    if (nranks <= 0 || rank < 0 || rank >= nranks || segments <= 0 || batch <= 0 || nheads <= 0 || state_elems <= 0 ||
        batch * nheads > 65535 || nranks * segments > 2147483647LL)
        return fail(SSD_B200_EINVAL, "bad state_prefix_all dimensions");
    if (rank_stride < batch * segments * nheads * state_elems || logp_stride < batch * segments * nheads)
        return fail(SSD_B200_EINVAL, "state_prefix_all: a rank's block is smaller than its (b, S, h) records");
    if (outer && (!outer_logp || outer_n <= 0 || outer_n > 65535 || outer_rank < 0 || outer_rank >= outer_n ||
                  outer_stride < batch * nheads * state_elems || outer_logp_stride < batch * nheads))
        return fail(SSD_B200_EINVAL, "state_prefix_all: bad outer (per-rank) summaries");
    dim3 g((unsigned)((state_elems + 255) / 256), (unsigned)(batch * nheads));
    cudaStream_t st = (cudaStream_t)stream;
    SSD_LAUNCH(ssd::prof::K_PREFIX, st, ssd::simt::state_prefix_all_kernel<<<g, 256, 0, st>>>(
        pieces, logp, edge, out, total, total_logp, (int)nranks, (int)rank, (int)segments, (int)nheads, (size_t)state_elems,
        (size_t)rank_stride, (size_t)logp_stride, reverse, outer, outer_logp, (int)outer_n, (int)outer_rank,
        (size_t)outer_stride, (size_t)outer_logp_stride));
    CUDA_LAUNCH_CHECK("state_prefix_all");
    return 0;
}

}  // extern "C"
