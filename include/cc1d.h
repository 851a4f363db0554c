/*
 * cc1d.h — C ABI of the B200 (sm_100a) causal depthwise conv1d kernels.
 *
 * Every entry point takes a plain-old-data parameter block and a CUDA stream,
 * launches on the *current* device, allocates nothing, never synchronises and
 * returns an int status (CC1D_OK == 0).  All strides are in ELEMENTS (not bytes)
 * and are 64-bit.  Pointers are device pointers unless stated otherwise.
 *
 * Each entry point replaces one host function + kernel family of the reference
 * (Dao-AILab/causal-conv1d v1.6.1); the replaced interface is cited above it.
 */
#ifndef CC1D_H_
#define CC1D_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Opaque stream handle: pass a cudaStream_t (0 == legacy default stream). */
typedef void *cc1d_stream_t;

typedef enum cc1d_dtype {
    CC1D_F32 = 0,
    CC1D_F16 = 1,
    CC1D_BF16 = 2
} cc1d_dtype;

typedef enum cc1d_status {
    CC1D_OK = 0,
    CC1D_ERR_NULL = 1,          /* a required pointer is NULL                        */
    CC1D_ERR_DTYPE = 2,         /* dtype enum out of range                           */
    CC1D_ERR_WIDTH = 3,         /* width not in {2,3,4}                              */
    CC1D_ERR_SHAPE = 4,         /* negative size / inconsistent sizes                */
    CC1D_ERR_STRIDE = 5,        /* neither the channel nor the seqlen stride is 1    */
    CC1D_ERR_CL_DIM = 6,        /* channel-last needs dim % 8 == 0                   */
    CC1D_ERR_CL_STRIDE = 7,     /* channel-last needs batch/seqlen strides % 8 == 0  */
    CC1D_ERR_LAYOUT = 8,        /* seq_idx / states given with channel-first x       */
    CC1D_ERR_STATE_STRIDE = 9,  /* a state tensor needs channel stride 1             */
    CC1D_ERR_STATE_LEN = 10,    /* conv_state_len < width - 1                        */
    CC1D_ERR_WORKSPACE = 11,    /* workspace missing or too small                    */
    CC1D_ERR_ALIGN = 12,        /* pointer not aligned for its element type          */
    CC1D_ERR_TOO_LARGE = 13,    /* problem exceeds an internal index range           */
    CC1D_ERR_LAUNCH = 14,       /* the CUDA launch itself failed (see cudaGetLastError) */
    CC1D_ERR_SCRATCH_LIMIT = 15, /* problem needs more than the built-in scratch of cc1d_bwd_noalloc */
    CC1D_ERR_SCRATCH_ADDRESS = 16, /* cc1d_bwd_noalloc could not look up its built-in scratch on this device */
    CC1D_ERR_CAPTURE = 17,      /* first cc1d_bwd_noalloc call on a device made inside a stream capture */
    CC1D_ERR_SEQ_IDX_STATES = 18, /* seq_idx given together with initial/final states (use cc1d_prefill_varlen) */
    CC1D_ERR_PHASE = 19         /* cc1d_bwd_params.phase not in {0, 1, 2}                 */
} cc1d_status;

/* ---------------------------------------------------------------------------
 * Forward.  Replaces causal_conv1d_fwd() (csrc/causal_conv1d.cpp:149-258) and
 * the kernels behind it (csrc/causal_conv1d_fwd.cu:46-137 channel-first,
 * :205-348 channel-last); the block mirrors ConvParamsBase
 * (csrc/causal_conv1d.h:9-54).
 *
 *   out[b,c,t] = act(bias[c] + sum_w weight[c,w] * x[b,c,t-(width-1-w)])
 *
 * Layout rule (csrc/causal_conv1d.cpp:176): channel-last iff
 * x_c_stride == 1 && x_l_stride > 1, otherwise channel-first (x_l_stride == 1).
 * seq_idx, initial_states and final_states are channel-last only, and seq_idx
 * excludes the state tensors (the reference's Python layer asserts the same,
 * causal_conv1d/causal_conv1d_interface.py:27-33): under seq_idx the positions
 * before the first token belong to no sequence, so a state could never
 * contribute; the combination is rejected with CC1D_ERR_SEQ_IDX_STATES —
 * cc1d_prefill_varlen is the call for packed sequences with states.
 * ------------------------------------------------------------------------- */
typedef struct cc1d_fwd_params {
    int32_t itype;            /* cc1d_dtype of x, out, states                   */
    int32_t wtype;            /* cc1d_dtype of weight and bias                  */
    int32_t width;            /* 2, 3 or 4                                      */
    int32_t silu;             /* 0: identity, 1: SiLU                           */
    int64_t batch, dim, seqlen;

    const void *x;            /* (batch, dim, seqlen)                           */
    int64_t x_batch_stride, x_c_stride, x_l_stride;
    const void *weight;       /* (dim, width)                                   */
    int64_t weight_c_stride, weight_width_stride;
    const void *bias;         /* (dim,) contiguous, or NULL                     */
    void *out;                /* (batch, dim, seqlen), same layout class as x   */
    int64_t out_batch_stride, out_c_stride, out_l_stride;

    const int32_t *seq_idx;   /* (batch, seqlen) contiguous int32, or NULL      */
    const void *initial_states; /* (batch, dim, width-1), c stride 1, or NULL   */
    int64_t initial_states_batch_stride, initial_states_c_stride, initial_states_l_stride;
    void *final_states;       /* (batch, dim, width-1), c stride 1, or NULL     */
    int64_t final_states_batch_stride, final_states_c_stride, final_states_l_stride;
} cc1d_fwd_params;

int cc1d_fwd(const cc1d_fwd_params *p, cc1d_stream_t stream);

/* Ranks that exchange their weight gradients inside cc1d_bwd (see cc1d_bwd_params.peers).
 * peer_base[r]: address, valid on THIS device, of rank r's exchange buffer —
 * cc1d_peer_allreduce_buffer_bytes(world, capacity) bytes of peer-mapped device memory per
 * rank, zero-filled once, used by nothing else (in particular not by cc1d_peer_allreduce:
 * the two lay their lines out differently).  capacity >= dim * (width + 1).
 * A wait for a peer is bounded: spin_limit polls (0: the default, about half a second; a poll
 * sleeps ~0.25 us, so size it to the largest skew between ranks the job can have).  When it
 * runs out *status is set to 1 and the elements of dweight / dbias that could not be completed
 * are set to NaN, so a caller that never reads the status still cannot train on them. */
#define CC1D_MAX_PEERS 16
typedef struct cc1d_peer_group {
    int32_t world, rank;
    int64_t capacity;
    void *peer_base[CC1D_MAX_PEERS];
    int32_t *status;              /* device int32, zero-filled by the caller */
    uint32_t spin_limit;          /* polls before a wait gives up; 0: default */
    uint32_t reserved0;
} cc1d_peer_group;

/* ---------------------------------------------------------------------------
 * Backward.  Replaces causal_conv1d_bwd() (csrc/causal_conv1d.cpp:260-463) and
 * its kernels (csrc/causal_conv1d_bwd.cu:53-259 channel-first, :329-589
 * channel-last); the block mirrors ConvParamsBwd (csrc/causal_conv1d.h:56-88).
 *
 * dweight / dbias are fp32.  They are produced by a fixed-order reduction
 * (warp shuffle tree -> per-CTA partial rows in `workspace` -> one finishing
 * kernel), never by float atomics, so results are bitwise run-to-run
 * reproducible — the behaviour the reference only offers under
 * CAUSAL_CONV1D_DETERMINISTIC=1 (csrc/causal_conv1d.cpp:21-28,388-462).
 * With accumulate != 0 the finishing kernel adds to the existing contents of
 * dweight/dbias (the reference's contract: the caller zero-fills them,
 * causal_conv1d/cpp_functions.py:134-137); with accumulate == 0 it overwrites.
 * ------------------------------------------------------------------------- */
typedef struct cc1d_bwd_params {
    int32_t itype, wtype, width, silu;
    int64_t batch, dim, seqlen;

    const void *x;
    int64_t x_batch_stride, x_c_stride, x_l_stride;
    const void *weight;
    int64_t weight_c_stride, weight_width_stride;
    const void *bias;         /* may be NULL                                    */
    const void *dout;         /* same layout class as x; beside a channel-last x it
                                 may also be channel-first (l stride 1, 16-bit types,
                                 c / batch strides % 8 == 0, 16-byte aligned): read in
                                 place, no re-layout copy (the reference copies,
                                 csrc/causal_conv1d.cpp:297-298)                 */
    int64_t dout_batch_stride, dout_c_stride, dout_l_stride;
    void *dx;                 /* same layout class as x                         */
    int64_t dx_batch_stride, dx_c_stride, dx_l_stride;
    float *dweight;           /* (dim, width) fp32                              */
    int64_t dweight_c_stride, dweight_width_stride;
    float *dbias;             /* (dim,) fp32 contiguous, or NULL                */
    int32_t accumulate;       /* see above                                      */
    int32_t reserved0;

    const int32_t *seq_idx;
    const void *initial_states;
    int64_t initial_states_batch_stride, initial_states_c_stride, initial_states_l_stride;
    const void *dfinal_states;   /* (batch, dim, width-1), any strides, or NULL */
    int64_t dfinal_states_batch_stride, dfinal_states_c_stride, dfinal_states_l_stride;
    void *dinitial_states;       /* (batch, dim, width-1), c stride 1, or NULL  */
    int64_t dinitial_states_batch_stride, dinitial_states_c_stride, dinitial_states_l_stride;

    void *workspace;          /* >= cc1d_bwd_workspace_bytes() bytes, 16-B aligned, need not be zeroed */
    size_t workspace_bytes;

    /* NULL, or the ranks of a batch-sharded backward: the finishing kernel then also sums
     * dweight / dbias over all ranks through peer memory (one kernel does the last local
     * reduction and the exchange), every rank ending with the same bits.  No counterpart in
     * the reference. */
    const cc1d_peer_group *peers;

    /* 0: the whole backward.  1: only the main kernel (dx, dinitial_states, partial rows left
     * in `workspace`).  2: only the finishing kernel (partial rows -> dweight / dbias, and the
     * exchange over `peers`); same parameter block and workspace as the phase-1 call, on any
     * stream ordered after it.  Splitting lets the exchange between ranks run beside the next
     * kernels of the compute stream instead of in front of them. */
    int32_t phase;
    int32_t reserved1;
} cc1d_bwd_params;

/* Bytes of scratch cc1d_bwd needs for this problem (host-only arithmetic).
 * Returns 0 on invalid parameters. */
size_t cc1d_bwd_workspace_bytes(const cc1d_bwd_params *p);
int cc1d_bwd(const cc1d_bwd_params *p, cc1d_stream_t stream);

/* ---------------------------------------------------------------------------
 * Backward for callers that cannot allocate.  No counterpart in the reference
 * (its host code always allocates through PyTorch).
 *
 * Some hosts of this library have no way to hand cc1d_bwd a workspace: code that
 * runs where device allocation is forbidden or would stall (inside a region that
 * must not touch the allocator, a plugin whose host owns all device memory, a
 * latency-critical loop that may not call cudaMalloc).  For them this entry point
 * does the same work as cc1d_bwd with the partial-sum scratch taken from a fixed
 * buffer of CC1D_NOALLOC_SCRATCH_BYTES that lives inside the library image: every
 * GPU that loads libcc1d.so holds that much device memory until the process
 * exits.  p->workspace and p->workspace_bytes are ignored; x, dout, dx, dweight,
 * dbias and the state tensors are still the caller's.
 *
 *  - A problem whose partial rows (for the tiling that these pointers and
 *    strides select; never more than cc1d_bwd_workspace_bytes()) exceed the
 *    buffer is rejected with CC1D_ERR_SCRATCH_LIMIT and nothing is launched.
 *  - It calls no cudaMalloc / cudaFree / allocating library routine.  The first
 *    call on each device looks up the buffer's device address (one
 *    cudaGetSymbolAddress, with that device current); make that first call
 *    outside any stream capture — inside one it is refused with
 *    CC1D_ERR_CAPTURE (a failed lookup: CC1D_ERR_SCRATCH_ADDRESS).
 *  - All calls share the one buffer and it keeps the previous call's contents.
 *    Nothing in it has to start at zero (every slot that is read was written
 *    earlier in the same call), but two calls that overlap on the GPU (different
 *    streams, or different host threads without ordering) race on it: keep calls
 *    on one device ordered.
 * ------------------------------------------------------------------------- */
#define CC1D_NOALLOC_SCRATCH_BYTES (8u * 1024u * 1024u)
int cc1d_bwd_noalloc(const cc1d_bwd_params *p, cc1d_stream_t stream);

/* ---------------------------------------------------------------------------
 * Decode-step state update.  Replaces causal_conv1d_update()
 * (csrc/causal_conv1d.cpp:465-557) and causal_conv1d_update_kernel
 * (csrc/causal_conv1d_update.cu:23-114).  conv_state is updated in place.
 * cache_seqlens != NULL selects the circular-buffer mode;
 * conv_state_indices != NULL gathers the state row per batch entry, a negative
 * index marks a padded entry: its outputs are zero and no state is touched.
 * ------------------------------------------------------------------------- */
typedef struct cc1d_update_params {
    int32_t itype, wtype, width, silu;
    int64_t batch, dim, seqlen;

    const void *x;            /* (batch, dim, seqlen), any strides              */
    int64_t x_batch_stride, x_c_stride, x_l_stride;
    const void *weight;
    int64_t weight_c_stride, weight_width_stride;
    const void *bias;
    void *out;                /* (batch, dim, seqlen), any strides              */
    int64_t out_batch_stride, out_c_stride, out_l_stride;

    void *conv_state;         /* (entries, dim, conv_state_len), any strides    */
    int64_t conv_state_len;
    int64_t conv_state_batch_stride, conv_state_c_stride, conv_state_l_stride;
    const int32_t *cache_seqlens;       /* (batch,) or NULL                     */
    const int32_t *conv_state_indices;  /* (batch,) or NULL                     */
} cc1d_update_params;

int cc1d_update(const cc1d_update_params *p, cc1d_stream_t stream);

/* ---------------------------------------------------------------------------
 * Variable-length "last tokens -> conv state" gather.  Replaces the Triton
 * kernel _causal_conv1d_varlen_states and its wrapper
 * (causal_conv1d/causal_conv1d_varlen.py:8-32, :35-64):
 *   n = min(state_len, cu[b+1]-cu[b]);
 *   states[b, :, state_len-n:] = x[cu[b+1]-n : cu[b+1], :].T ; the rest is 0.
 * ------------------------------------------------------------------------- */
typedef struct cc1d_varlen_states_params {
    int32_t itype;
    int32_t cu_seqlens_is_int64;  /* 0: int32 cu_seqlens, 1: int64              */
    int64_t total_tokens, dim, batch, state_len;
    const void *x;                /* (total_tokens, dim)                         */
    int64_t x_l_stride, x_c_stride;
    const void *cu_seqlens;       /* (batch + 1,) contiguous                     */
    void *states;                 /* (batch, dim, state_len)                     */
    int64_t states_batch_stride, states_c_stride, states_l_stride;
} cc1d_varlen_states_params;

int cc1d_varlen_states(const cc1d_varlen_states_params *p, cc1d_stream_t stream);

/* ---------------------------------------------------------------------------
 * Packed variable-length prefill with per-sequence conv states (an additive
 * extension: the reference has no single call for it — its forward forbids
 * seq_idx together with initial_states / final_states,
 * causal_conv1d/causal_conv1d_interface.py:27-33, and per-sequence states come
 * from a second pass, causal_conv1d/causal_conv1d_varlen.py:35-64).
 *
 * x is a channel-last pack of nseq sequences, (total_tokens, dim) with channel
 * stride 1; sequence s owns tokens [cu_seqlens[s], cu_seqlens[s+1]).  With
 * r = state_indices ? state_indices[s] : s  and  S = state_len:
 *
 *   prefix_s = has_initial_state[s] (or has_initial_state == NULL and
 *              initial_states != NULL) ? initial_states[r] : zeros(dim, S)
 *   out[cu[s] : cu[s+1]]  = causal conv (+ bias, + SiLU) of x[cu[s] : cu[s+1]]
 *                           whose left context is the last width-1 entries of prefix_s
 *                           — what causal_conv1d_ref(x_s, initial_states=...) returns;
 *   final_states[r]       = last S entries of [prefix_s | x_s]
 *                           — causal_conv1d_varlen_states when there is no prefix,
 *                           the reference's final_states when S == width-1.
 *
 * Tokens at or after cu_seqlens[nseq] and tokens whose seq_idx is negative output
 * zero.  A negative state index gives the sequence a zero prefix and stores no
 * final state.  final_states may alias initial_states (in-place pool update) as
 * long as no two sequences name the same row.
 *
 * seq_idx (total_tokens,) int32 must be the sequence number of every token
 * (cc1d_seq_idx_from_cu_seqlens fills it).  Two launches on the stream: the
 * forward kernel, then a boundary kernel that recomputes the first width-1
 * outputs of each prefixed sequence and writes the final states.
 * ------------------------------------------------------------------------- */
typedef struct cc1d_prefill_varlen_params {
    int32_t itype, wtype, width, silu;
    int64_t total_tokens, dim, nseq, state_len;

    const void *x;                  /* (total_tokens, dim), channel stride 1       */
    int64_t x_l_stride;
    const void *weight;
    int64_t weight_c_stride, weight_width_stride;
    const void *bias;
    void *out;                      /* (total_tokens, dim), channel stride 1       */
    int64_t out_l_stride;

    const int32_t *seq_idx;         /* (total_tokens,)                             */
    const int32_t *cu_seqlens;      /* (nseq + 1,) non-decreasing, cu[0] == 0      */
    const int32_t *state_indices;   /* (nseq,) or NULL                             */
    const uint8_t *has_initial_state; /* (nseq,) 0/1 or NULL                       */

    const void *initial_states;     /* (rows, dim, state_len), channel stride 1, or NULL */
    int64_t initial_states_batch_stride, initial_states_l_stride;
    void *final_states;             /* (rows, dim, state_len), channel stride 1, or NULL */
    int64_t final_states_batch_stride, final_states_l_stride;
} cc1d_prefill_varlen_params;

int cc1d_prefill_varlen(const cc1d_prefill_varlen_params *p, cc1d_stream_t stream);

/* seq_idx[t] = s for cu_seqlens[s] <= t < cu_seqlens[s+1], -1 for t >= cu_seqlens[nseq].
 * The reference's callers build this tensor in PyTorch (tests/test_causal_conv1d.py:437-447). */
int cc1d_seq_idx_from_cu_seqlens(const int32_t *cu_seqlens, int64_t nseq, int64_t total_tokens,
                                 int32_t *seq_idx, cc1d_stream_t stream);

/* Human-readable text for a status code (static storage, never NULL). */
const char *cc1d_status_str(int status);

/* ---------------------------------------------------------------------------
 * One-shot all-reduce (sum) of a small fp32 vector over NVLink peer memory — the
 * exchange step of the batch-sharded backward (dweight | dbias of all ranks).  No
 * counterpart in the reference, which has no multi-GPU code.
 *
 * Every rank calls it with the same world and count, its own rank, and either the same
 * explicit epoch (1, 2, 3, ... one per collective) or epoch 0 on every call: then the
 * kernel numbers the collectives itself with a counter in the rank's exchange buffer,
 * which makes a captured CUDA graph replayable (do not mix the two modes on one buffer).  peer_base[r] is the address, valid on THIS
 * device, of rank r's exchange buffer: cc1d_peer_allreduce_buffer_bytes(world, count)
 * bytes of peer-mapped device memory per rank, zero-filled once before the first call
 * and not touched by anything else.  The kernel stores this rank's vector, stamped with
 * the epoch, into every rank's buffer, polls (bounded) its own buffer for all ranks'
 * vectors and adds them in rank order, so all ranks end with the same bits.
 * dst may equal src.  count must be a multiple of 4; src and dst 16-byte aligned.
 * Polls are bounded (spin_limit polls of ~0.25 us; 0: the default, about half a second —
 * size it to the largest skew between ranks the job can have).  If one runs out (a peer
 * never arrived) *status is set to 1 and every element of dst that could not be completed
 * is set to NaN; the call itself still returns CC1D_OK (it cannot know).  Read the status
 * before using the sums for anything that cannot be undone (an optimizer step).  Calls of
 * one communicator must be ordered on each rank.
 * ------------------------------------------------------------------------- */
typedef struct cc1d_peer_allreduce_params {
    int32_t world, rank;
    uint32_t epoch;
    uint32_t spin_limit;          /* polls before a wait gives up; 0: default */
    int64_t count;
    const float *src;
    float *dst;
    void *peer_base[CC1D_MAX_PEERS];
    int32_t *status;              /* device int32, zero-filled by the caller */
} cc1d_peer_allreduce_params;

size_t cc1d_peer_allreduce_buffer_bytes(int32_t world, int64_t count);
int cc1d_peer_allreduce(const cc1d_peer_allreduce_params *p, cc1d_stream_t stream);

/* Health check (no reference counterpart).  The TMA kernels wait on shared-memory barriers
 * with an iteration limit instead of forever; a wait that runs out makes the kernel stop early
 * and raise a device-side flag.  This call SYNCHRONISES the current device, returns 0 when no
 * wait has run out since the last call (bit 0: forward, bit 1: backward; -1: the flags could
 * not be read) and clears the flags.  A non-zero answer means outputs written since the last
 * call are incomplete.  Never expected in practice; not for the hot path. */
int cc1d_wait_expired(void);

/* Library ABI version: bumped when a parameter block changes layout or entry points are added. */
int cc1d_abi_version(void);

#ifdef __cplusplus
}
#endif
#endif /* CC1D_H_ */
