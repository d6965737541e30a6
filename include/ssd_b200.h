/*
 * ssd_b200 -- C ABI of the B200 (sm_100a) SSD chunked scan, forward and backward.
 *
 * This is the drop-in boundary for the reference's fused SSD scan operator
 * (reference paths are relative to its r2/dhammic-ai directory):
 *
 *   fused_ssd_scan(x, A, B, C, chunk_size, initial_states, cache)   src/kernels/ssd_scan.py:539-583
 *   FusedSSDScan.forward / .backward                                src/kernels/ssd_scan.py:441-533
 *   _ssd_forward_impl (the algorithm)                               src/kernels/ssd_scan.py:330-421
 *
 * The reference has no native code; its operator is Python over Triton and
 * cuBLAS.  A maintainer binds these entry points from Python with ctypes
 * (dhammic-ai_b200/_cabi.py is such a binding).  Conventions:
 *
 *   - plain pointers and sizes only; every pointer is a DEVICE pointer on the
 *     current CUDA device unless stated otherwise; tensors are dense row-major
 *     in the layouts given below;
 *   - `stream` is a cudaStream_t passed as void* (NULL = legacy default stream);
 *     all work is enqueued on it and nothing synchronises the host;
 *   - every function returns 0 on success or a negative SSD_B200_E* code and
 *     never throws, aborts or traps; ssd_b200_last_error() gives a
 *     thread-local message for the last failure on the calling thread;
 *   - the library allocates nothing: the caller provides outputs and one
 *     workspace of ssd_b200_workspace_bytes() bytes, 256-byte aligned.
 *
 * Symbols: b batch, T seqlen, h heads, p headdim, n d_state, g groups
 * (g divides h; head j uses group j / (h/g)), l chunk, c = T / l.
 */
#ifndef SSD_B200_H_
#define SSD_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define SSD_B200_ABI_VERSION 3

enum {
    SSD_B200_OK = 0,
    SSD_B200_EINVAL = -1,       /* bad shape, null pointer, bad flag combination      */
    SSD_B200_EUNSUPPORTED = -2, /* shape outside what the kernels cover               */
    SSD_B200_EWORKSPACE = -3,   /* workspace missing, too small or misaligned         */
    SSD_B200_ECUDA = -4,        /* a CUDA runtime call or launch failed               */
    SSD_B200_EDEVICE = -5       /* a kernel reported a bounded wait that ran out      */
};

enum { SSD_B200_F32 = 0, SSD_B200_BF16 = 1 };

enum { SSD_B200_PASS_FWD = 0, SSD_B200_PASS_BWD = 1 };

/* Which kernels run.  AUTO picks the tcgen05 tensor-core path when the shape
 * and dtype allow it (bf16; p = 64; n = 128; T a multiple of 128) and the
 * fp32 SIMT path otherwise; the other two force a path (for tests). */
enum { SSD_B200_PATH_AUTO = 0, SSD_B200_PATH_SIMT = 1, SSD_B200_PATH_TC = 2 };

/* Partial passes used by the sequence-parallel schedule (each rank holds a contiguous slice of the
 * sequence and only per-rank states cross NVLink):
 *   SSD_B200_FWD_STATES_ONLY  forward: write final_state (and a_cumsum, logdecay_total) only; y may be NULL.
 *   SSD_B200_BWD_DINIT_ONLY   backward: from dy, C, a_cumsum (and dfinal, NULL = zero) alone write dinit, the
 *                             gradient of the initial state; every other output may be NULL.
 *   SSD_B200_FWD_AUX_VALID    forward, tensor-core path, with `states` given: the per-position arrays in `states` were
 *                             already written by an earlier forward call on the same dt / a / skip (e.g. the STATES_ONLY
 *                             pass of the same slice, which takes `states` too and fills only that part) and are
 *                             reused instead of rebuilt.  Combine with cumsum_is_input to reuse a_cumsum as well. */
enum { SSD_B200_FWD_STATES_ONLY = 1, SSD_B200_FWD_AUX_VALID = 2 };
enum { SSD_B200_BWD_DINIT_ONLY = 1 };

typedef struct ssd_b200_shape {
    int32_t abi_version; /* SSD_B200_ABI_VERSION                                      */
    int32_t dtype;       /* storage of x, B, C, y, dy, dx, dB, dC                      */
    int32_t a_dtype;     /* storage of the per-position log-decay `a` (when given)     */
    int32_t path;        /* SSD_B200_PATH_*                                            */
    int64_t batch, seqlen, nheads, headdim, dstate, ngroups, chunk;
} ssd_b200_shape;

/*
 * Forward.  Replaces _ssd_forward_impl (src/kernels/ssd_scan.py:330-421) and,
 * with dt/A_head/D given, also the caller's input products and D skip
 * (src/mamba_base_engine.py:170-173, :187).
 *
 * Three ways to give the decay and the input scaling:
 *   (1) operator form:  a != NULL, dt == A_head == D == NULL:  X = x, log-decay = a   (b,T,h)
 *   (2) Mamba-2 form:   a == NULL, dt (b,T,h) fp32, A_head (h) fp32, D (h) fp32 or NULL:
 *                       X = x * dt, log-decay = dt * A_head, y += D * x
 *   (3) scaled operator form (tensor-core path only): a != NULL and dt (b,T,h) fp32 != NULL, A_head == D == NULL:
 *                       X = x * dt, log-decay = a, and with skip (b,T,h) fp32 != NULL  y += skip * x
 *       (a per-position input weight and a per-position skip coefficient: what the Mamba-3 style block's
 *       single-scan form needs, src/mamba_base_engine.py:170-187, without materialising x * weight).
 *
 *   x (b,T,h,p)  B,C (b,T,g,n)  init (b,h,p,n) fp32 or NULL  ->  y (b,T,h,p), final_state (b,h,p,n) fp32
 *   Log-decays are expected to be <= 0 (the reference's parametrisation, A = -exp(.), guarantees it); the kernels
 *   do not clamp positive values the way the reference's exp-clamp does at +20.
 *   a_cumsum (b,h,c,l) fp32: within-chunk inclusive cumulative log-decay; written unless
 *   cumsum_is_input != 0, in which case it is read as given (the reference's cached call,
 *   src/kernels/ssd_scan.py:364-373).
 */
typedef struct ssd_b200_fwd_args {
    ssd_b200_shape shape;
    const void *x;
    const void *a;
    const float *dt;
    const float *A_head;
    const float *D;
    const void *B;
    const void *C;
    const float *init;
    void *y;
    float *final_state;
    float *a_cumsum;
    int32_t cumsum_is_input;
    int32_t flags;       /* SSD_B200_FWD_* */
    void *workspace;
    size_t workspace_bytes;
    void *states; /* optional output, ssd_b200_states_bytes() bytes: the recurrent state entering every
                     128-position tile and the per-position decay arrays of the tile kernels, in the layout
                     the backward wants.  Passing the same buffer to ssd_b200_bwd (same inputs) saves it the
                     state walk and the rebuild of those arrays; NULL = do not save. */
    float *logdecay_total; /* optional output (b,h) fp32: the sum of the sequence's log-decays per (batch, head),
                              i.e. log of the factor by which the whole sequence scales an incoming state */
    float *ysq;            /* optional output, tensor-core path only (must be NULL otherwise), T a multiple of 128:
                              (b, T/128, h, 2, 128) fp32, sum over one half (32 values) of the head's row of y^2 for
                              position 128 * tile + i, stored [b][tile][h][half][i].  Summed over h and half it is the
                              row's sum of squares that the RMS norm after the scan needs
                              (ssd_b200_rmsnorm_fwd_presummed), which then reads y once instead of twice. */
    const float *skip;     /* form (3) only: per-position skip coefficient (b,T,h) fp32, or NULL */
} ssd_b200_fwd_args;

/*
 * Backward.  Replaces FusedSSDScan.backward (src/kernels/ssd_scan.py:468-533): given dy
 * (b,T,h,p) and optionally dfinal (b,h,p,n) fp32 it writes
 *   dx (b,T,h,p), dB, dC (b,T,g,n) in storage dtype, dinit (b,h,p,n) fp32 (optional), and
 *   operator form : da (b,T,h) fp32 -- gradient of the per-position log-decay; skipped (may be
 *                   NULL) when cumsum_is_input != 0, matching the reference, whose cached call
 *                   returns no decay gradient (src/kernels/ssd_scan.py:494-500, :533);
 *   Mamba-2 form  : ddt (b,T,h) fp32, dA_head (h) fp32, dD (h) fp32 (dD only when D != NULL);
 *   scaled operator form: da (b,T,h) fp32, ddt (b,T,h) fp32 = gradient of the input weight (sum_p dX x), and with
 *                   skip given dskip (b,T,h) fp32 = sum_p dy x; dx already contains skip * dy.
 * a_cumsum is the tensor the forward produced (or was given).
 */
typedef struct ssd_b200_bwd_args {
    ssd_b200_shape shape;
    const void *x;
    const void *a;
    const float *dt;
    const float *A_head;
    const float *D;
    const void *B;
    const void *C;
    const float *init;
    const float *a_cumsum;
    const void *dy;
    const float *dfinal;
    void *dx;
    void *dB;
    void *dC;
    float *da;
    float *ddt;
    float *dA_head;
    float *dD;
    float *dinit;
    int32_t cumsum_is_input;
    int32_t flags;       /* SSD_B200_BWD_* */
    void *workspace;
    size_t workspace_bytes;
    const void *states; /* optional: what the forward wrote into its `states`; NULL = recompute */
    const float *skip;  /* scaled operator form: the forward's skip (b,T,h) fp32, or NULL */
    float *dskip;       /* scaled operator form with skip: (b,T,h) fp32 */
} ssd_b200_bwd_args;

/* ABI version of the loaded library (compare with SSD_B200_ABI_VERSION). */
int ssd_b200_abi_version(void);

/* Message for the last failure on this thread ("" if none).  The pointer stays valid until
 * the next failing call on the same thread. */
const char *ssd_b200_last_error(void);

/* Bytes of workspace one call of the given pass needs for this shape (0 on a bad shape). */
size_t ssd_b200_workspace_bytes(const ssd_b200_shape *shape, int pass);

/* Bytes of the optional `states` buffer for this shape; 0 when the resolved path does not use one
 * (then `states` must be NULL). */
size_t ssd_b200_states_bytes(const ssd_b200_shape *shape);

/* Which path AUTO resolves to for this shape: SSD_B200_PATH_SIMT or SSD_B200_PATH_TC
 * (negative code on a bad shape).  Host-only, needs no GPU. */
int ssd_b200_resolve_path(const ssd_b200_shape *shape);

int ssd_b200_fwd(const ssd_b200_fwd_args *args, void *stream);
int ssd_b200_bwd(const ssd_b200_bwd_args *args, void *stream);

/*
 * Forward without a caller workspace.  This entry point has no counterpart in the reference.
 *
 * Same arguments and results as ssd_b200_fwd, except that `workspace` and `workspace_bytes` are
 * ignored: the scratch comes from a fixed array of ssd_b200_static_scratch_bytes() (64 MiB) that
 * is part of the library's device code.  It is meant for hosts that cannot obtain device memory
 * of their own -- a plugin under a framework that hands it only input and output pointers, or a
 * process whose device memory was reserved up front and where cudaMalloc is off limits -- and so
 * could never supply the buffer ssd_b200_fwd needs.  It calls no cudaMalloc, cudaFree or other
 * allocating routine (keep the profiling hooks off, they create events).
 *
 *   - Limit: a shape whose forward scratch (ssd_b200_workspace_bytes(shape, SSD_B200_PASS_FWD))
 *     exceeds the array is refused with SSD_B200_EWORKSPACE and a message naming both sizes.
 *   - Every GPU on which the library is loaded holds the array until the process exits.
 *   - Every call looks the array's device address up with cudaGetSymbolAddress for the context that
 *     is current on the calling thread (nothing is cached, so a device reset or a second context on
 *     the same GPU cannot leave a stale address behind).  The first lookup on a device loads the
 *     library's device code there: make the first call before any stream capture.
 *   - All calls on a device share the one array.  It keeps whatever the previous call left; the
 *     kernels overwrite what they read and the one word that must start at zero is cleared on
 *     the stream at the start of each call.  Two calls that overlap on the GPU (different
 *     streams, or different host threads) race on it: serialise them.
 */
int ssd_b200_fwd_static_scratch(const ssd_b200_fwd_args *args, void *stream);
size_t ssd_b200_static_scratch_bytes(void);

/*
 * Optional check after a call (it synchronises `stream`): the tensor-core kernels bound every
 * wait on a barrier; if one ran out, the kernel finished anyway, set a status word at the start
 * of the workspace and this returns SSD_B200_EDEVICE.  `workspace` is the buffer the call was given;
 * NULL means the built-in array of ssd_b200_fwd_static_scratch on the current device.  No counterpart
 * in the reference.
 */
int ssd_b200_device_status(const ssd_b200_shape *shape, const void *workspace, void *stream);

/*
 * Self-test of the error path above (no counterpart in the reference): launches one warp that waits `polls`
 * polls on a barrier nothing arrives at, gives up and sets the status word at the start of `workspace` (>= 4
 * bytes, device memory) the way the tile kernels do; ssd_b200_device_status(shape, workspace, stream) for a
 * tensor-core shape then returns SSD_B200_EDEVICE.  Nothing faults or hangs and the context stays usable.
 */
int ssd_b200_selftest_bounded_wait(void *workspace, int32_t polls, void *stream);

/*
 * The reference operator also returns its decay masks as a cache
 * (src/kernels/ssd_scan.py:420, :465; shapes pinned by tests/kernels/test_ssd_scan.py:107-110).
 * This builds them from a_cumsum on demand:
 *   L (b,h,c,l,l)          = exp(clamp(cum_i - cum_j, -20, 20)) for i >= j, exp(-20) above
 *   decay_chunk (b,h,c+1,c+1) = the same construction over the zero-padded chunk totals
 * in `dtype` storage.  Either output may be NULL.
 */
int ssd_b200_materialize_cache(const ssd_b200_shape *shape, const float *a_cumsum, void *L,
                               void *decay_chunk, int32_t dtype, void *stream);

/*
 * Sequence-parallel state prefix (no counterpart in the reference, which has no multi-GPU path; it builds on
 * the operator's initial_states / final_state contract, src/kernels/ssd_scan.py:395-397, :410, and on
 * d final_state in / d initial_states out, :468, :530-533).
 *
 * The sequence is cut into nranks * segments consecutive pieces, piece g = r * segments + s.  Every piece has a
 * summary (what it adds to the state after it for a zero state before it -- ssd_b200_fwd with
 * SSD_B200_FWD_STATES_ONLY -- or, in reverse, what it adds to the gradient of the state before it --
 * ssd_b200_bwd with SSD_B200_BWD_DINIT_ONLY) and a total log-decay (logdecay_total of the forward).  All of
 * them are already in THIS GPU's memory (e.g. after an all_gather): rank r's summaries at
 * pieces + r * rank_stride as (batch, segments, h, state_elems) fp32, its log-decays at
 * logp + r * logp_stride as (batch, segments, h) fp32 (strides in floats).  One launch writes into
 * out (batch, segments, h, state_elems), for each of the `segments` pieces of `rank`,
 *   reverse == 0:  the state entering the piece,       acc_0 = edge,    acc_{g+1} = exp(logp_g) acc_g + pieces_g
 *   reverse != 0:  the state gradient leaving the piece, acc_last = edge, acc_{g-1} = exp(logp_g) acc_g + pieces_g
 * with edge (batch, h, state_elems) the caller's initial state / final-state gradient, or NULL for zero.  Every
 * piece is read once.  The outputs are in the layout ssd_b200_fwd / _bwd take as init / dfinal when the
 * segments run as batch entries (entry = batch index * segments + s).  Optional outputs (NULL = skip; `out` may
 * be NULL when only these are wanted): total (batch, h, state_elems) = acc after the last of rank's pieces has been
 * folded in, total_logp (batch, h) = sum of the log-decays of rank's own pieces -- with nranks = 1 these are the
 * summary and log-decay of the rank's whole slice, i.e. what the ranks exchange (one state per rank, not one per
 * segment).  With `outer` != NULL the walk is preceded by such slice summaries of the other ranks: outer + q *
 * outer_stride is rank q's (batch, h, state_elems) summary, outer_logp + q * outer_logp_stride its (batch, h)
 * log-decay, outer_n ranks with this one at outer_rank; forward folds those before it, reverse those behind it, and
 * `edge` lies beyond all of them.  That makes the rank-level and the segment-level prefix one launch (pass nranks = 1,
 * rank = 0 and the local segments as `pieces`).
 */
int ssd_b200_state_prefix_all(const float *pieces, const float *logp, const float *edge, float *out, float *total,
                              float *total_logp, int64_t nranks, int64_t rank, int64_t segments, int64_t batch,
                              int64_t nheads, int64_t state_elems, int64_t rank_stride, int64_t logp_stride,
                              int32_t reverse, const float *outer, const float *outer_logp, int64_t outer_n,
                              int64_t outer_rank, int64_t outer_stride, int64_t outer_logp_stride, void *stream);

/*
 * Exchange of the per-rank summaries by direct stores into the other GPUs' memory over NVLink peer access (no
 * counterpart in the reference; an alternative to an NCCL all_gather for the 2 MiB blocks above, whose cost is
 * latency).  Every rank owns a receive buffer of nranks slots and a row of nranks arrival counters (uint32, zero at
 * start); peer_bufs[q] / peer_flags[q] are DEVICE arrays holding rank q's buffer and counters as mapped into this
 * process (entry `rank` = the own ones).  The host side that allocates, maps (CUDA IPC) and owns them is
 * dhammic-ai_b200/distributed.py (PeerStoreComm).
 *   exchange_push:   copies src[0, n) into every rank's buffer at float offset dst_offset (n, dst_offset multiples
 *                    of 4; src 16-byte aligned) with plain stores -- no TMA, no multicast.
 *   exchange_arrive: (after the push, same stream) stores `epoch` into counter `rank` of every peer and waits until
 *                    every peer's counter here has reached `epoch` (epochs grow by one per exchange).  The wait polls
 *                    at most max_polls times per peer; if it runs out, *status (device memory) is set to 3 and the
 *                    kernel returns -- nothing hangs, the gathered data is invalid and the host must check status.
 */
/* CUDA IPC plumbing for the buffers above (host-side, no kernels).  export: the 64-byte handle of the allocation that
 * contains `ptr` and ptr's byte offset inside it.  import: maps that allocation into this process with the CURRENT
 * device as the accessor (peer access to the owning GPU is enabled as part of the open) and returns its base; the
 * same allocation must be imported once per process.  close: unmaps. */
int ssd_b200_ipc_export(const void *ptr, unsigned char *handle64, int64_t *offset);
int ssd_b200_ipc_import(const unsigned char *handle64, void **base_out);
int ssd_b200_ipc_close(void *base);
/* Lets kernels of the current device access memory of `peer_device` (cudaDeviceEnablePeerAccess; already enabled is
 * fine).  SSD_B200_EUNSUPPORTED when the two devices are not peers. */
int ssd_b200_enable_peer_access(int32_t peer_device);
int ssd_b200_exchange_push(const float *src, int64_t n, float *const *peer_bufs, int64_t nranks, int64_t dst_offset,
                           void *stream);
int ssd_b200_exchange_arrive(unsigned int *const *peer_flags, int64_t rank, int64_t nranks, uint32_t epoch,
                             int32_t *status, uint32_t max_polls, void *stream);

/*
 * Element-wise kernels of the Mamba-3 style variant (no counterpart in the reference's operator file: its
 * block does these steps with tensor arithmetic, src/mamba_base_engine.py:128-187).  The block's two scan
 * calls  SSD(x gamma, a, Br, Cr) + SSD(shift(x) beta, a, shift(Br), Cr)  collapse into ONE scan
 *     Y = SSD(x w, a, Br, Cr) + (D - u s) x,   w = lam dt + u,  u[t] = (1 - lam[t+1]) dt[t+1] (0 at the end),
 * s = <B, C> per group (the rotation preserves it), a = dt A_head.
 *   prologue_fwd: cum = -cumsum_T(raw_angles) (b,T,h,n/2); Br, Cr = rope(B, cum), rope(C, cum) (b,T,h,n);
 *                 sdot = s (b,T,g); dA = a; and either xw = x w (xw != NULL) or, with xw == NULL, the per-position
 *                 coefficients w_out = w and skip_out = D - u s (b,T,h) for the scan's scaled operator form, which
 *                 then applies them itself (x is not read here).
 *   skip_fwd:     y = y_scan + (D - u s) x   (y may be y_scan; D may be NULL).
 *   prologue_bwd: from the scan's gradients dBr, dCr and dw = <dxw, x>, dyx = <dy, x> per (b,t,h):  dB, dC (b,T,g,n)
 *                 (rotation undone, heads of a group summed, plus the s term) and d raw_angles.  With dxw != NULL it
 *                 first forms dx = dxw w + (D - u s) dy, dw and dyx itself; with dxw == NULL dw and dyx are inputs
 *                 (the scaled operator form's ddt and dskip) and x, dy, dx are not touched.
 * x, B, C and the tensor outputs are in shape->dtype; raw_angles / d_raw_angles in angles_dtype (fp32 or shape->dtype;
 * the cumulative angle is fp32 either way); dt, lam, A_head, D, dA, sdot, cum, dw, dyx, w_out, skip_out are fp32.
 * segsum_ws: b * ceil(T/128) * h * n/2 floats of scratch; dcum_ws: (b,T,h,n/2) fp32 scratch.
 */
int ssd_b200_m3_prologue_fwd(const ssd_b200_shape *shape, const void *x, const float *dt, const float *lam,
                             const float *A_head, const void *B, const void *C, const void *raw_angles,
                             int32_t angles_dtype, void *xw, float *dA, void *Br, void *Cr, float *sdot, float *cum,
                             float *segsum_ws, const float *D, float *w_out, float *skip_out, void *stream);
int ssd_b200_m3_skip_fwd(const ssd_b200_shape *shape, const void *y_scan, const void *x, const float *D, const float *dt,
                         const float *lam, const float *sdot, void *y, void *stream);
/* Chain rule of the single-scan form on the (b,T,h) fp32 tensors, after ssd_b200_m3_prologue_bwd (dw, dyx) and the
 * scan backward (da): with v[t] = dw[t] - s[t] dyx[t] (s = sdot of the head's group) and v[-1] = 0,
 *   dlam = (dw - v[t-1]) dt,   ddt = dw lam + v[t-1] (1 - lam) + da A_head,
 *   dA_head[h] = sum_{b,t} da dt,   dD[h] = sum_{b,t} dyx  (dD may be null).
 * The sums over (b,t) are two-stage with a fixed order (deterministic).  ws: ssd_b200_m3_chain_ws_floats(shape)
 * floats of scratch.  In the reference these steps are autograd through the block's element-wise expressions
 * (src/mamba_base_engine.py:150-187). */
size_t ssd_b200_m3_chain_ws_floats(const ssd_b200_shape *shape);
int ssd_b200_m3_chain_bwd(const ssd_b200_shape *shape, const float *dw, const float *dyx, const float *sdot,
                          const float *dt, const float *lam, const float *da, const float *A_head, float *dlam,
                          float *ddt, float *dA_head, float *dD, float *ws, void *stream);
int ssd_b200_m3_prologue_bwd(const ssd_b200_shape *shape, const void *x, const void *dy, const float *dt,
                             const float *lam, const float *D, const void *B, const void *C, const float *cum,
                             const float *sdot, const void *dxw, const void *dBr, const void *dCr, void *dx, float *dw,
                             float *dyx, void *dB, void *dC, void *d_raw_angles, int32_t angles_dtype, float *dcum_ws,
                             float *segsum_ws, void *stream);

/*
 * The two element-wise operators that feed the scan in the reference's block, stand-alone:
 *   rope:      y = rotation of the interleaved pairs (x[2m], x[2m+1]) by angles[m]     src/kernels/rope.py:228-325
 *              (FusedRoPE / fused_rope).  x, y, dy, dx (B,T,H,D) in `dtype`; angles fp32 (B,T,1,D/2) when
 *              broadcast_h, else (B,T,H,D/2); dangles fp32 in the angles' shape (summed over heads when broadcast).
 *   trapezoid: dt = softplus(dt_raw + dt_bias), dA = dt * -exp(A_log), beta = (1 - sigmoid(lam_raw)) dt exp(dA),
 *              gamma = sigmoid(lam_raw) dt                                     src/kernels/trapezoidal.py:220-335
 *              (FusedTrapezoidal / fused_trapezoidal).  Tensors are (rows, H) in `dtype`; dt_bias, A_log,
 *              d_dt_bias, d_A_log are fp32 (H); ws: ssd_b200_trapezoid_ws_floats(rows, H) floats of scratch.
 */
int ssd_b200_rope_fwd(int32_t dtype, int64_t B, int64_t T, int64_t H, int64_t D, int32_t broadcast_h, const void *x,
                      const float *angles, void *y, void *stream);
int ssd_b200_rope_bwd(int32_t dtype, int64_t B, int64_t T, int64_t H, int64_t D, int32_t broadcast_h, const void *x,
                      const float *angles, const void *dy, void *dx, float *dangles, void *stream);
size_t ssd_b200_trapezoid_ws_floats(int64_t rows, int64_t H);
int ssd_b200_trapezoid_fwd(int32_t dtype, int64_t rows, int64_t H, const void *dt_raw, const void *lam_raw,
                           const float *dt_bias, const float *A_log, void *dt, void *dA, void *beta, void *gamma,
                           void *stream);
int ssd_b200_trapezoid_bwd(int32_t dtype, int64_t rows, int64_t H, const void *dt_raw, const void *lam_raw,
                           const float *dt_bias, const float *A_log, const void *g_dt, const void *g_dA,
                           const void *g_beta, const void *g_gamma, void *d_dt_raw, void *d_lam_raw, float *d_dt_bias,
                           float *d_A_log, float *ws, void *stream);

/*
 * RMS norm over the last dimension, optionally gated (the step after the scan in the reference's block):
 *     out = x * rsqrt(mean(x^2) + eps) * weight  [* silu(z) when z != NULL]
 * src/kernels/rmsnorm.py:154-230 (FusedRMSNorm / fused_rmsnorm); with z it is the block's `norm(y) * silu(z)`
 * (src/mamba_base_engine.py:189-191) in one pass.  x, z, out, dout, dx, dz are (rows, D) in `dtype`; weight,
 * dweight fp32 (D); rstd fp32 (rows), written by the forward and read by the backward; ws:
 * ssd_b200_rmsnorm_ws_floats(rows, D) floats of scratch.
 */
size_t ssd_b200_rmsnorm_ws_floats(int64_t rows, int64_t D);
/* The same forward with the row's sum of squares given as partial sums written by the scan's forward (`ysq` of
 * ssd_b200_fwd_args; rows = b * T with T a multiple of 128, D = nheads * 64): one pass over x (and z). */
int ssd_b200_rmsnorm_fwd_presummed(int32_t dtype, int64_t rows, int64_t D, float eps, const void *x, const float *weight,
                                   const void *z, const float *ysq, int64_t nheads, void *out, float *rstd, void *stream);
int ssd_b200_rmsnorm_fwd(int32_t dtype, int64_t rows, int64_t D, float eps, const void *x, const float *weight,
                         const void *z, void *out, float *rstd, void *stream);
int ssd_b200_rmsnorm_bwd(int32_t dtype, int64_t rows, int64_t D, const void *x, const float *weight, const void *z,
                         const void *dout, const float *rstd, void *dx, void *dz, float *dweight, float *ws,
                         void *stream);

/*
 * Measurement hooks (no counterpart in the reference).  ssd_b200_launch_count() is the number of
 * kernels this library has launched in the process.  With profiling enabled every launch is
 * bracketed by CUDA events on its stream; ssd_b200_profile_read() waits for them, adds their
 * durations (ms) and launch counts per kernel slot into ms[n] / launches[n]
 * (n >= ssd_b200_profile_kernels()) and clears the record.  For single-threaded benchmark use.
 */
long long ssd_b200_launch_count(void);
int ssd_b200_profile_enable(int on);
int ssd_b200_profile_kernels(void);
const char *ssd_b200_profile_kernel_name(int idx);
int ssd_b200_profile_read(float *ms, long long *launches, int n);

#ifdef __cplusplus
}
#endif
#endif /* SSD_B200_H_ */
