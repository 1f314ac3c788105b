/* mok_b200: C-ABI of the B200-native MoE-layer hot path.
 *
 * Drop-in boundary for the `_C` extension of cursor/mixture-of-kittens: every
 * entry point below replaces one function that the reference binds in
 * csrc/bindings.cu:6-94 (the pybind11 module `_C`), with at::Tensor arguments
 * flattened to raw device pointers + sizes.  No PyTorch type appears here.
 *
 * Conventions
 *   - every function returns MOKB_OK (0) or a negative error code and leaves a
 *     message retrievable with mokb_last_error() (thread-local);
 *   - all pointers are device pointers on the current CUDA device unless the
 *     name ends in `_host`; tensors are contiguous, row-major;
 *   - `stream` is a cudaStream_t passed as void*; work is enqueued, never
 *     synchronised: no entry point blocks the host.  The layer entry points also use two
 *     streams of their own per device (the pulls, at high priority, and the token-wise MXFP8
 *     copies, at low priority), forked from and joined back into `stream` with events inside the
 *     call, so that to the caller everything is ordered on `stream`;
 *   - "peer pointer lists" (`*_ptrs_host`) are host arrays of `ep_size` device
 *     addresses, index = EP rank, as produced by a symmetric-memory rendezvous
 *     (mok/functional.py:224 of the reference);
 *   - the caller allocates every output (the reference's callee-allocates
 *     convention, csrc/megakernel/forward.cuh:345-368, lives in the Python shim);
 *   - `status` points to FOUR device int32 words.  Kernels set word 0 to a
 *     MOKB_ST_* code instead of trapping or spinning for ever (the reference traps
 *     on schedule overflow, csrc/scheduler.cuh:86, and spins without bound,
 *     csrc/utils.cuh:274-277); after MOKB_ST_FLAG_TIMEOUT words 1..3 say which wait
 *     ran out (1 = a GEMM on a dispatch window, 2 = a down tile on its gate/up tiles,
 *     3 = combine on a GEMM window; the counter's index; value seen << 16 | target).
 *     The words are only ever written when something went wrong; the caller zeroes them.
 */
#ifndef MOK_B200_H
#define MOK_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define MOKB_OK 0
#define MOKB_ERR_INVALID (-1)   /* bad argument */
#define MOKB_ERR_CUDA (-2)      /* a CUDA runtime/driver call failed */
#define MOKB_ERR_UNSUPPORTED (-3)

#define MOKB_MAX_EP 64          /* EP sizes 1..64 (the reference: 1,4,8,16,32,64; mok/functional.py:156) */

/* device status codes */
#define MOKB_ST_OK 0
#define MOKB_ST_SCHEDULE_OVERFLOW 1   /* padded rows exceed schedule_capacity */
#define MOKB_ST_BARRIER_TIMEOUT 2     /* a peer never arrived at barrier_all */
#define MOKB_ST_PIPELINE_TIMEOUT 3    /* an mbarrier wait inside a GEMM ran out */
#define MOKB_ST_MACROBATCH_OVERFLOW 4 /* reserved: every layer entry point splits the rows into macrobatches */
#define MOKB_ST_FLAG_TIMEOUT 5        /* a wait on a counter that another kernel or CTA raises ran out (2 s) */
#define MOKB_ST_BAD_INDEX 6           /* a schedule entry names a route outside [0, tokens * topk): the row was skipped.
                                       * Words 1..3: 1 pull / 2 push kernel / 3 GEMM epilogue push, the row, the index */

const char* mokb_last_error(void);
/* Compute capability major*10+minor of the current device, or a negative error. */
int mokb_device_arch(void);
int mokb_sm_count(void);
/* sizeof() of {mokb_fwd_bf16_args, mokb_bwd_bf16_args, mokb_gemm_args}: lets a binding verify its struct layout. */
int mokb_struct_sizes(int* out, int n);
/* Number of kernels this library has launched in this process (all threads). */
unsigned long long mokb_launch_count(void);
/* Launch timeline, a diagnostic with no counterpart in the reference (its benchmarks time whole passes,
 * benchmarks/utils.py:66-110).  After mokb_trace_begin(stream) every launcher of this library brackets what it
 * enqueues with two timing events (up to 8192 launches; one host thread).  mokb_trace_end synchronises the
 * device, stops recording and writes one line per launcher call, "tag arg stream_no begin_ms end_ms" with times
 * relative to the begin call and streams numbered in order of first use; it returns the number of bytes the
 * full text needs (write again with a larger buffer if that exceeds cap), or -1 on a CUDA error. */
int mokb_trace_begin(void* stream);
long long mokb_trace_end(char* out, size_t cap);

/* ---- route all-gather: replaces `_C.all_gather_top_experts`
 * (csrc/utils.cuh:191-249).  Copies this rank's [numel] int32 routes into slot
 * `rank` of every peer's [ep_size, numel] buffer with plain peer stores. */
int mokb_all_gather_top_experts(const int32_t* top_experts, const uint64_t* gather_buffer_ptrs_host,
                                int ep_size, int rank, int64_t numel, void* stream);

/* ---- device barrier over all EP ranks: replaces `_C.barrier_all`
 * (csrc/utils.cuh:251-299).  `target` (device int32, local) grows by ep_size per
 * call; each rank adds 1 to every rank's barrier word and waits, with a bounded
 * spin, until its own word reaches the target. */
int mokb_barrier_all(const uint64_t* barrier_ptrs_host, int ep_size, int rank, int32_t* target,
                     int32_t* status, void* stream);
/* How long a rank waits for its peers before giving up with MOKB_ST_BARRIER_TIMEOUT (default 10 s). */
int mokb_set_barrier_timeout_ms(int ms);

/* ---- routing schedule: replaces `_C.schedule` (csrc/scheduler.cuh:149-183).
 * topk_all [ep_size, num_local_tokens, topk] int32 -> peer_rank [capacity],
 * peer_token_idx [capacity], num_tokens [1], tokens_per_expert [num_local_experts].
 * Padding rows get peer_rank = peer_token_idx = -1.  `scratch` must hold
 * mokb_schedule_scratch_bytes() bytes; it needs no initialisation. */
size_t mokb_schedule_scratch_bytes(int ep_size, int num_local_experts);
int mokb_schedule(const int32_t* topk_all, int ep_size, int num_local_tokens, int topk,
                  int num_local_experts, int schedule_capacity, int rank,
                  int32_t* peer_rank, int32_t* peer_token_idx, int32_t* num_tokens,
                  int32_t* tokens_per_expert, void* scratch, int32_t* status, void* stream);

/* ---- routing schedule without device allocation.  No counterpart in the reference.
 * For callers that cannot allocate device memory around the call -- a host framework that
 * owns the device heap through its own pool, a step loop where cudaMalloc's implicit
 * synchronisation is unaffordable, a process that commits all its memory at start-up:
 * same inputs, outputs and result as mokb_schedule, but the work area is a fixed array
 * inside the library image (4 MiB + 16 KiB, resident on every GPU that loads the library,
 * until the process exits) instead of caller-provided scratch.  The caller still passes all
 * inputs and outputs.  The call makes no cudaMalloc / cudaFree and uses no allocating routine.
 *   - Limit: ep_size * num_local_experts <= MOKB_SCHEDULE_NOALLOC_MAX_EXPERTS; beyond it the
 *     call fails with MOKB_ERR_INVALID and a message that names the limit.
 *   - The first call on a device looks up the array's device address (once per device, with
 *     that device current); make that first call before any stream capture begins.
 *   - All calls on a device share the one array and find in it what the last call left; the
 *     entry point clears the part that must start at zero.  Two calls whose kernels overlap
 *     on the GPU (different streams, or different host threads) race on it: serialise them. */
#define MOKB_SCHEDULE_NOALLOC_MAX_EXPERTS 1024
int mokb_schedule_noalloc(const int32_t* topk_all, int ep_size, int num_local_tokens, int topk,
                          int num_local_experts, int schedule_capacity, int rank,
                          int32_t* peer_rank, int32_t* peer_token_idx, int32_t* num_tokens,
                          int32_t* tokens_per_expert, int32_t* status, void* stream);

/* ---- MXFP8 quantiser: replaces `_C.mxfp8_quantize` (csrc/mxfp8.cuh:234-278).
 * x [E, M, N] bf16 (E = 1 for a matrix); outputs may be NULL pairwise:
 * fp8 [E, M, N] + sc [E*M/128, N/128, 32, 16]; fp8_t [E, N, M] + sc_t [E*N/128, M/128, 32, 16]. */
int mokb_mxfp8_quantize(const void* x_bf16, int64_t E, int64_t M, int64_t N,
                        void* x_fp8, void* x_sc, void* x_fp8_t, void* x_sc_t, void* stream);

/* ---- epilogues: replace `_C.fwd_epilogue` / `_C.bwd_epilogue` (csrc/utils.cuh:12-189). */
int mokb_fwd_epilogue(const void* y_shared, const void* combine_buffer, const float* topk_weights,
                      void* output, int64_t num_local_tokens, int64_t hidden, int topk, void* stream);
int mokb_bwd_epilogue(const void* d_x_shared, const void* d_x_routed_buffer, void* d_x,
                      int64_t num_local_tokens, int64_t hidden, int topk, void* stream);

/* ---- the fused layer: replace `_C.dispatch_mlp_swiglu_combine_{fwd,bwd}_bf16`
 * (csrc/megakernel/entrypoints.cuh:101-164, 425-503; host launchers
 * forward.cuh:432-540, backward.cuh:684-873) and `_C.recompute_forward_context_bf16`
 * (recompute_forward_context.cuh).  One struct carries what the reference passes
 * positionally; fields are named after the reference's arguments. */
typedef struct {
    /* sizes */
    int ep_size, ep_rank;
    int num_local_tokens, hidden, intermediate, num_local_experts, topk;
    int schedule_capacity, macrobatch_size, minibatch_size, num_comm_sms;
    int has_swiglu_limit;
    float swiglu_limit;
    /* schedule */
    const int32_t* peer_rank;
    const int32_t* peer_token_idx;
    const int32_t* num_tokens;
    const int32_t* tokens_per_expert;
    /* symmetric buffers (host arrays of ep_size device addresses) */
    const uint64_t* x_ptrs_host;              /* [T, H] bf16 per rank */
    const uint64_t* combine_ptrs_host;        /* [T*K, H] bf16 per rank (forward output) */
    /* weights */
    const void *w_shared_gate, *w_shared_up, *w_shared_down;   /* [I,H] [I,H] [H,I] bf16 */
    const void *w_routed_gate, *w_routed_up, *w_routed_down;   /* [E_l,I,H] [E_l,I,H] [E_l,H,I] bf16 */
    /* outputs, caller-allocated (ops.py:432-441 of the reference) */
    void *x_routed;                            /* [MB, H] */
    void *gate_shared, *up_shared, *hidden_shared;   /* [T, I] */
    void *gate_routed, *up_routed, *hidden_routed;   /* [MB, I] */
    void *y_shared;                            /* [T, H] */
    void *y_routed;                            /* [MB, H], optional: the rows go to the peers' combine buffers from the down
                                                  GEMM's epilogue; given, they are stored here as well (the reference's
                                                  staging buffer, read by nothing afterwards) */
    /* scratch: mokb_layer_scratch_bytes() bytes, no initialisation needed */
    void* scratch;
    int32_t* status;
    int skip_down_combine;                     /* 1 = recompute_forward_context */
} mokb_fwd_bf16_args;

typedef struct {
    int ep_size, ep_rank;
    int num_local_tokens, hidden, intermediate, num_local_experts, topk;
    int schedule_capacity, macrobatch_size, minibatch_size, num_comm_sms;
    int has_swiglu_limit;
    float swiglu_limit;
    const int32_t* peer_rank;
    const int32_t* peer_token_idx;
    const int32_t* num_tokens;
    const int32_t* tokens_per_expert;
    const uint64_t* d_y_ptrs_host;             /* [T, H] bf16 per rank */
    const uint64_t* d_x_routed_ptrs_host;      /* [T*K, H] bf16 per rank (output) */
    const uint64_t* router_weight_ptrs_host;   /* [T, K] f32 per rank */
    const uint64_t* d_router_weight_ptrs_host; /* [T, K] f32 per rank (output) */
    const uint64_t* x_ptrs_host;               /* [T, H] bf16 per rank */
    const void *w_shared_gate, *w_shared_up, *w_shared_down;
    const void *w_routed_gate, *w_routed_up, *w_routed_down;
    /* saved forward context (macrobatch 0) */
    const void *x_routed, *gate_shared, *gate_routed, *up_shared, *up_routed, *hidden_shared, *hidden_routed;
    /* outputs (ops.py:1169-1184 of the reference) */
    void *d_x_shared, *d_x_routed;             /* [T,H] [MB,H]; d_x_routed optional, as y_routed in the forward */
    void *d_gate_shared, *d_gate_routed, *d_up_shared, *d_up_routed;   /* [T,I] [MB,I] */
    void *d_hidden_shared, *d_hidden_routed;   /* [T,I] [MB,I] */
    void *d_y_routed;                          /* [MB,H] */
    void *d_w_shared_gate, *d_w_routed_gate, *d_w_shared_up, *d_w_routed_up;
    void *d_w_shared_down, *d_w_routed_down;
    void* scratch;                             /* mokb_layer_scratch_bytes() */
    int32_t* status;
} mokb_bwd_bf16_args;

size_t mokb_layer_scratch_bytes(int schedule_capacity, int num_local_experts, int macrobatch_size);
int mokb_dispatch_mlp_swiglu_combine_fwd_bf16(const mokb_fwd_bf16_args* args, void* stream);
int mokb_dispatch_mlp_swiglu_combine_bwd_bf16(const mokb_bwd_bf16_args* args, void* stream);

/* ---- the fused layer in MXFP8: replace `_C.dispatch_mlp_swiglu_combine_{fwd,bwd}_mxfp8` and
 * `_C.recompute_forward_context_mxfp8` (csrc/megakernel/entrypoints.cuh:11-96, 169-332; host launchers
 * forward.cuh:296-428, backward.cuh:448-679).  Routed experts run in block-scaled E4M3, the shared expert
 * in BF16.  E4M3 tensors are passed as byte pointers; every `*_sc` is a packed scale tensor
 * [rows/128, cols/128, 32, 16] for the tensor it follows.  "work" buffers are caller-allocated and need
 * no initialisation; their contents after the call are unspecified. */
typedef struct {
    int ep_size, ep_rank;
    int num_local_tokens, hidden, intermediate, num_local_experts, topk;
    int schedule_capacity, macrobatch_size, minibatch_size, num_comm_sms;
    int has_swiglu_limit;
    float swiglu_limit;
    const int32_t* peer_rank;
    const int32_t* peer_token_idx;
    const int32_t* num_tokens;
    const int32_t* tokens_per_expert;
    const uint64_t* x_ptrs_host;
    const uint64_t* combine_ptrs_host;
    const void *w_shared_gate, *w_shared_up, *w_shared_down;                  /* bf16 */
    const void *w_routed_gate, *w_routed_gate_sc;                             /* [E_l, I, H] quantised along H */
    const void *w_routed_up, *w_routed_up_sc;
    const void *w_routed_down, *w_routed_down_sc;                             /* [E_l, H, I] quantised along I */
    /* outputs (ops.py:265-278 of the reference) */
    void *x_fp8_t, *x_sc_t;                                                   /* [H, MB]: x_routed^T quantised along tokens */
    void *gate_shared, *up_shared, *hidden_shared;                            /* [T, I] bf16 */
    void *gate_fp8, *gate_sc, *up_fp8, *up_sc;                                /* [MB, I] */
    void *hidden_fp8_t, *hidden_sc_t;                                         /* [I, MB] */
    void *y_shared, *y_routed;                                                /* [T, H], [MB, H] bf16 */
    /* work */
    void *x_routed;                                                           /* [MB, H] bf16 */
    void *x_fp8, *x_sc;                                                       /* [MB, H] */
    void *hidden_fp8, *hidden_sc;                                             /* [MB, I] */
    void* scratch;                                                            /* mokb_layer_scratch_bytes() */
    int32_t* status;
    int skip_down_combine;                                                    /* 1 = recompute_forward_context */
} mokb_fwd_mxfp8_args;

typedef struct {
    int ep_size, ep_rank;
    int num_local_tokens, hidden, intermediate, num_local_experts, topk;
    int schedule_capacity, macrobatch_size, minibatch_size, num_comm_sms;
    int has_swiglu_limit;
    float swiglu_limit;
    const int32_t* peer_rank;
    const int32_t* peer_token_idx;
    const int32_t* num_tokens;
    const int32_t* tokens_per_expert;
    const uint64_t* d_y_ptrs_host;
    const uint64_t* d_x_routed_ptrs_host;
    const uint64_t* router_weight_ptrs_host;
    const uint64_t* d_router_weight_ptrs_host;
    const uint64_t* x_ptrs_host;
    const void *w_shared_gate, *w_shared_up, *w_shared_down;                  /* bf16 */
    const void *w_routed_gate_t, *w_routed_gate_t_sc;                         /* [E_l, H, I] = W_gate^T quantised along I */
    const void *w_routed_up_t, *w_routed_up_t_sc;
    const void *w_routed_down_t, *w_routed_down_t_sc;                         /* [E_l, I, H] = W_down^T quantised along H */
    /* saved forward context; the routed tensors are overwritten when later macrobatches are replayed */
    void *x_fp8_t, *x_sc_t;
    const void *gate_shared;
    void *gate_fp8, *gate_sc;
    const void *up_shared;
    void *up_fp8, *up_sc;
    const void *hidden_shared;
    void *hidden_fp8_t, *hidden_sc_t;
    /* outputs (ops.py:903-921 of the reference) */
    void *d_x_shared, *d_x_routed;                                            /* [T, H], [MB, H] bf16 */
    void *d_gate_shared, *d_gate_fp8, *d_gate_sc;                             /* [T, I] bf16; [MB, I] */
    void *d_up_shared, *d_up_fp8, *d_up_sc;
    void *d_hidden_shared, *d_hidden_routed;                                  /* [T, I], [MB, I] bf16 */
    void *d_y_fp8, *d_y_sc;                                                   /* [MB, H] */
    void *d_w_shared_gate, *d_w_routed_gate, *d_w_shared_up, *d_w_routed_up, *d_w_shared_down, *d_w_routed_down;   /* bf16 */
    /* work */
    void *d_y_routed;                                                         /* [MB, H] bf16 */
    void *d_y_fp8_t, *d_y_sc_t;                                               /* [H, MB] */
    void *d_gate_fp8_t, *d_gate_sc_t, *d_up_fp8_t, *d_up_sc_t;                /* [I, MB] */
    void *partials;                                                           /* [MB, I/128] f32 */
    /* replay of macrobatches 1.. (the saved context holds macrobatch 0; the backward rebuilds the later ones into
     * the context buffers, which it therefore overwrites, ops.py:785-791 of the reference).  Required only when
     * schedule_capacity > macrobatch_size; null otherwise. */
    const void *w_routed_gate, *w_routed_gate_sc, *w_routed_up, *w_routed_up_sc;   /* forward weights, quantised along H */
    void *x_routed;                                                           /* [MB, H] bf16 */
    void *x_fp8, *x_sc;                                                       /* [MB, H] */
    void *hidden_fp8, *hidden_sc;                                             /* [MB, I] */
    void* scratch;
    int32_t* status;
} mokb_bwd_mxfp8_args;

int mokb_dispatch_mlp_swiglu_combine_fwd_mxfp8(const mokb_fwd_mxfp8_args* args, void* stream);
int mokb_dispatch_mlp_swiglu_combine_bwd_mxfp8(const mokb_bwd_mxfp8_args* args, void* stream);
/* sizeof() of {mokb_fwd_mxfp8_args, mokb_bwd_mxfp8_args, mokb_gemm_fp8_args}. */
int mokb_struct_sizes_mxfp8(int* out, int n);

/* ---- building blocks, exported for tests and micro-benchmarks.  They are the
 * kernels the two layer calls above are made of. */

/* Grouped GEMM D = A * B^T over row groups: rows [0, *num_rows) of A in blocks of
 * 128, block b using weight matrix group_of_block[b] (NULL = one group).
 *   mode 0: B [G, N, K] (K contiguous)            -> D [rows, N]
 *   mode 1: same as 0 with B = gate and B2 = up   -> D = gate, D2 = up, D3 = SwiGLU(gate, up), all [rows, N]
 *   mode 2: B [G, K, N] (N contiguous; "dgrad")   -> D [rows, N]; if A2/B2 given, D = A*B + A2*B2
 * Weight-gradient GEMM (mode 3): for each group g with rows [off[g], off[g+1]) of
 * A [rows, M] and B [rows, N]: D[g] [M, N] = A_g^T * B_g (zero if the group is empty).
 *   mode 4: mode 1 followed by the down projection of the same rows, D4 [rows, N2] = D3 * B3[g]^T with B3 [G, N2, N],
 *           in ONE persistent launch that walks the rows window by window (window_rows rows each): all gate/up tiles of
 *           a window, then all its down tiles -- the task order of the reference's forward megakernel
 *           (csrc/megakernel/forward.cuh:146-266).  N2 = 0 leaves the down projection out.
 * Counters (modes 0, 1, 2, 4; device int32 arrays that the caller zeroes; the reference's barrier_wait / barrier_arrive,
 * csrc/megakernel/utils.cuh:1-13, with a 2 s limit after which the kernel sets MOKB_ST_FLAG_TIMEOUT and exits):
 *   win_ready[w] -- awaited (>= win_ready_target) before the first A rows of window w (counted from row_begin) are read;
 *                   mokb_dispatch_rows_window adds 1 per block when its rows have landed;
 *   blk_done[b]  -- mode 4, required, [rows / 256 from row_begin]: the kernel's own count of finished gate/up tiles per
 *                   256-row block, awaited by its down tiles;
 *   win_done[w]  -- mode 4, optional: 8 arrivals per finished down tile of window w; mokb_combine_rows_window waits
 *                   for (rows of the window / 256) * (N2 / 256) * 8 of them before it reads D4. */
typedef struct {
    int mode;
    int rows_static;            /* row capacity of A and D; the row count when num_rows is NULL */
    int row_begin, row_end;     /* modes 0-2: only rows [row_begin, min(row_end, rows)) are computed; row_end = 0 means all.
                                   Both must be multiples of 256. */
    const int32_t* num_rows;    /* device, optional */
    const int32_t* group_of_block;   /* device [rows/128], optional */
    const int32_t* group_offsets;    /* device [G+1] (mode 3) */
    int G, M, N, K;             /* mode 0-2: N,K; mode 3: M,N */
    const void *A, *B, *A2, *B2;
    int lda, ldb;               /* row strides in elements */
    void *D, *D2, *D3;
    int ldd;
    int has_swiglu_limit;
    float swiglu_limit;
    int accumulate;             /* mode 3: D[g] += result (read, add in fp32, round to bf16); empty groups are left alone */
    int32_t* status;
    /* mode 4 and the counters */
    const void* B3;
    void* D4;
    int N2, ldb3, ldd4;
    int window_rows;
    const int32_t* win_ready;
    int win_ready_target;
    int32_t* blk_done;
    int32_t* win_done;
    /* push (modes 0, 2 and the down projection of mode 4): combine without a combine kernel
     * (dispatch_combine.cuh:152-266 of the reference pushes the rows from a staging buffer).  Row r of the result goes
     * to row push_idx[r] of rank push_rank[r]'s buffer (leading dimension ldd, mode 4: ldd4) with plain peer stores from
     * the GEMM's epilogue; rows whose rank is outside [0, push_ep_size) go nowhere.  With push_values, the first column
     * tile also writes push_value_ptrs[rank][push_idx[r]] = push_values[r] (router-weight gradients).  D (mode 4: D4)
     * may then be NULL; given, the rows are stored there as well. */
    const uint64_t* push_ptrs_host;
    int push_ep_size;
    const int32_t* push_rank;
    const int32_t* push_idx;
    const float* push_values;
    const uint64_t* push_value_ptrs_host;
    /* rows of each destination buffer (0 = unchecked): a push_idx outside [0, push_index_limit) is not stored anywhere and
     * sets MOKB_ST_BAD_INDEX -- a stale or foreign schedule must not become a store into a peer's memory */
    int64_t push_index_limit;
    /* mode 3, optional, device [G]: rows of group g from group_k_end[g] on (up to off[g+1]) are zero in A and B -- the
     * padding at the end of an expert's segment -- and are left out of the contraction, in steps of 64 rows */
    const int32_t* group_k_end;
} mokb_gemm_args;
int mokb_grouped_gemm_bf16(const mokb_gemm_args* args, void* stream);

/* Grouped MXFP8 GEMM (E4M3 data + one E8M0 scale per 32 elements of K, scales in the packed
 * [rows/128, K/128, 32, 16] layout the quantiser emits), fp32 accumulation, bf16 output.  Both operands
 * have the contraction axis contiguous (csrc/megakernel/grouped_gemm.cuh:183-237 of the reference).
 *   mode 0: D[rows,N] = A[rows,K] * B[g][N,K]^T, plus A2 * B2[g]^T into the same tile when A2 is given
 *   mode 1: D = A * B[g]^T and D2 = A * B2[g]^T in one pass (gate and up), N columns each
 *   mode 2: D[g][M,N] = A[M, cols_g] * B[N, cols_g]^T with cols_g = [off[g], off[g+1]) of the
 *           rows_static token columns of A [M, rows_static] and B [N, rows_static] (weight gradients).
 *           t_first: A and B hold the token columns [t_first, t_first + rows_static) of the row space that
 *           group_offsets refers to (a macrobatch of a longer schedule); offsets outside are not allowed.
 *           accumulate != 0 adds to the stored bf16 D (a group with an empty window then leaves D untouched
 *           instead of zeroing it).
 *   mode 3: the two products of mode 1 without the bf16 round trip: gate and up are rounded to bf16 in the
 *           epilogue, hidden = SwiGLU(gate, up) (clamped if has_swiglu_limit), and the kernel writes gate_q, up_q,
 *           hid_q [rows, N] E4M3 with scales along columns and hid_qt [N, t_rows] with scales along tokens: what
 *           mode 1 followed by the reference's SwiGLU + quantise pass produces (grouped_gemm.cuh:295-359,
 *           swiglu.cuh:38-207).  D and D2 are not used.
 *   mode 4: mode 3 followed by the down projection of the same rows, D [rows, N2] = hidden * B3[g]^T with B3 [G, N2, N]
 *           quantised along N, in ONE persistent launch, window by window -- mode 4 of mokb_grouped_gemm_bf16 in MXFP8,
 *           with the same counters (blk_done counts 16 arrivals per gate/up tile, win_done 16 per down tile) and the
 *           same push of the result rows to peers (modes 0 and 4; ldd is then the peers' leading dimension). */
typedef struct {
    int mode;
    int rows_static, row_begin, row_end;     /* as in mokb_gemm_args; multiples of 256 */
    const int32_t* num_rows;
    const int32_t* group_of_block;
    const int32_t* group_offsets;
    int G, M, N, K;
    const void *A, *A_sc, *B, *B_sc, *A2, *A2_sc, *B2, *B2_sc;
    void *D, *D2;
    int ldd;
    int t_first, accumulate;                 /* mode 2 only */
    void *gate_q, *gate_sc, *up_q, *up_sc, *hid_q, *hid_sc, *hid_qt, *hid_sct;   /* mode 3 only */
    int t_rows, has_swiglu_limit;
    float swiglu_limit;
    int32_t* status;
    /* mode 4, the counters and the push: as the fields of the same names in mokb_gemm_args */
    const void *B3, *B3_sc;
    int N2;
    int window_rows;
    const int32_t* win_ready;
    int win_ready_target;
    int32_t* blk_done;
    int32_t* win_done;
    const uint64_t* push_ptrs_host;
    int push_ep_size;
    const int32_t* push_rank;
    const int32_t* push_idx;
    const float* push_values;
    const uint64_t* push_value_ptrs_host;
    int64_t push_index_limit;      /* as in mokb_gemm_args */
    /* A launch with win_ready leaves this many SMs (0 = 2) to the kernels that produce the rows it waits for (the
     * reference sets whole SMs aside for communication: num_comm_sms).  The layer uses 2. */
    int reserve_sms;
} mokb_gemm_fp8_args;
int mokb_grouped_gemm_mxfp8(const mokb_gemm_fp8_args* args, void* stream);

/* Row gather from peers (dispatch, csrc/megakernel/dispatch_combine.cuh:1-150):
 * dst[i] = src_rank(peer_rank[i])[peer_token_idx[i] / row_divisor] for i < *num_rows;
 * rows with peer_rank < 0 are zero-filled.  If row_scale_ptrs_host is given, the row is
 * multiplied in fp32 by scale_rank[peer_token_idx[i]] and rounded to bf16, and the scale
 * is also written to row_scale_out[i] (0 for padding rows). */
int mokb_dispatch_rows(const uint64_t* src_ptrs_host, int ep_size, const int32_t* peer_rank,
                       const int32_t* peer_token_idx, const int32_t* num_rows, int max_rows,
                       int row_divisor, int64_t hidden, void* dst,
                       const uint64_t* row_scale_ptrs_host, float* row_scale_out, void* stream);
/* Row scatter to peers (combine, dispatch_combine.cuh:152-266):
 * dst_rank(peer_rank[i])[peer_token_idx[i]] = src[i]; optionally also
 * val_rank(peer_rank[i])[peer_token_idx[i]] = row_values[i] (router-weight gradients). */
int mokb_combine_rows(const void* src, const uint64_t* dst_ptrs_host, int ep_size,
                      const int32_t* peer_rank, const int32_t* peer_token_idx,
                      const int32_t* num_rows, int max_rows, int64_t hidden,
                      const float* row_values, const uint64_t* value_ptrs_host, void* stream);

/* The same two kernels on a row window [row_begin, min(row_end, *num_rows)), on `blocks` CTAs (0 = default), tied to a
 * GEMM that runs at the same time by counters instead of launch order (dispatch_combine.cuh:1-266 runs them as tasks of
 * the megakernel, synchronised through csrc/megakernel/utils.cuh:1-13):
 *   done_counter  -- optional; every block of the dispatch launch adds 1 once its rows have landed.  A GEMM given this
 *                    word as win_ready[w] with win_ready_target = the launch's block count (`blocks`, or
 *                    mokb_comm_default_blocks() when blocks is 0) starts window w only then.
 *   q_out, q_sc_out -- optional, together (hidden % 128 == 0, 32-byte aligned rows): the pulled (and scaled) rows also in
 *                    MXFP8, E4M3 [max_rows, hidden] + packed scales, quantised along the columns from the registers
 *                    they pass through (dispatch_combine.cuh:88-114); byte for byte what mokb_mxfp8_quantize gives.
 *   index_limit   -- routes per rank (tokens * topk; 0 = unchecked): a row whose peer_token_idx is outside [0, index_limit)
 *                    is treated as padding (pull: zeros; push: not stored) and sets MOKB_ST_BAD_INDEX in `status`, so
 *                    that a stale or foreign schedule cannot turn into an access outside a peer's buffer.  The layer
 *                    entry points always pass it.
 *   wait_counter  -- optional; the combine launch first waits (2 s at most, then MOKB_ST_FLAG_TIMEOUT in `status` and
 *                    no row is copied) until it holds ((rows of the window) / 256) * arrivals_per_row_block arrivals:
 *                    win_done[w] of a mode-4 GEMM with arrivals_per_row_block = (N2 / 256) * 8.  row_begin must be a
 *                    multiple of 256. */
int mokb_comm_default_blocks(void);
int mokb_dispatch_rows_window(const uint64_t* src_ptrs_host, int ep_size, const int32_t* peer_rank,
                              const int32_t* peer_token_idx, const int32_t* num_rows, int max_rows, int row_begin,
                              int row_end, int row_divisor, int64_t hidden, void* dst,
                              const uint64_t* row_scale_ptrs_host, float* row_scale_out, int blocks,
                              int32_t* done_counter, void* q_out, void* q_sc_out, int64_t index_limit, int32_t* status,
                              void* stream);
int mokb_combine_rows_window(const void* src, const uint64_t* dst_ptrs_host, int ep_size,
                             const int32_t* peer_rank, const int32_t* peer_token_idx,
                             const int32_t* num_rows, int max_rows, int row_begin, int row_end, int64_t hidden,
                             const float* row_values, const uint64_t* value_ptrs_host, int blocks,
                             const int32_t* wait_counter, int arrivals_per_row_block, int32_t* status, int64_t index_limit,
                             void* stream);

/* SwiGLU forward / backward on [rows, cols] bf16 (csrc/megakernel/swiglu.cuh:38-207, 209-566).
 * Backward also emits per-row sum(d_hidden * silu(g)*u) / w (w = row_scale[i], 1/w := 0 if w <= 0)
 * when row_grad_out is given. */
int mokb_swiglu_fwd(const void* gate, const void* up, void* hidden, const int32_t* num_rows, int64_t max_rows,
                    int64_t cols, int has_limit, float limit, void* stream);
int mokb_swiglu_bwd(const void* gate, const void* up, const void* d_hidden, void* d_gate, void* d_up,
                    const float* row_scale, float* row_grad_out, const int32_t* num_rows,
                    int64_t max_rows, int64_t cols, int has_limit, float limit, void* stream);

#ifdef __cplusplus
}
#endif
#endif
