// Shared device/host helpers for the sm_100a kernels of this library:
// error plumbing, bounded waits, and thin wrappers over the PTX the kernels
// are written in (mbarrier, TMA bulk tensor copies, tcgen05 MMA / TMEM).
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include "../../include/mok_b200.h"

namespace mokb {

// ---------------------------------------------------------------- host side
void set_error(const char* fmt, ...);
int cuda_fail(cudaError_t e, const char* what, const char* file, int line);

#define MOKB_CUDA(expr)                                                        \
    do {                                                                       \
        cudaError_t _e = (expr);                                               \
        if (_e != cudaSuccess) return ::mokb::cuda_fail(_e, #expr, __FILE__, __LINE__); \
    } while (0)

#define MOKB_REQUIRE(cond, ...)                                                \
    do {                                                                       \
        if (!(cond)) { ::mokb::set_error(__VA_ARGS__); return MOKB_ERR_INVALID; } \
    } while (0)

#define MOKB_TRY(expr)                                                         \
    do { int _r = (expr); if (_r != MOKB_OK) return _r; } while (0)

int sm_count();

// Kernels that run on the side streams beside a GEMM ask for the same shared-memory / L1 split as the GEMM (all
// shared memory).  An SM changes its split only when it is empty: blocks of a kernel with the default split that sit
// on every SM -- above all blocks that WAIT for the GEMM -- would keep its 197 KB CTAs from ever being placed.
template <class Kernel>
inline void share_sms_with_gemm(Kernel kernel) {
    static bool done = false;       // one flag per kernel type
    if (!done) {
        cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout, static_cast<int>(cudaSharedmemCarveoutMaxShared));
        done = true;
    }
}
// Launch timeline (diagnostic, off unless mokb_trace_begin was called): an object of this class in a launcher
// brackets everything the launcher enqueues on `stream` with two timing events.
class TraceScope {
public:
    TraceScope(cudaStream_t stream, const char* tag, int arg = 0);
    ~TraceScope();
private:
    int slot_;
    cudaStream_t stream_;
};
void note_launch(int n = 1);   // counts kernels launched by this library (reported by the benchmark)

// 2-D bf16/u8 tensor map with 128-byte swizzle: `inner` contiguous elements,
// `outer` rows of `row_stride_bytes`; box = box_inner x box_outer.
int make_tmap_2d(CUtensorMap* out, const void* base, int elem_bytes, uint64_t inner, uint64_t outer,
                 uint64_t row_stride_bytes, uint32_t box_inner, uint32_t box_outer);

// Row-window forms of dispatch / combine used by the layer to overlap them with the GEMMs:
// rows [row_begin, min(row_end, *num_rows)) only, on `blocks` CTAs of 128 threads (0 = default).
// `done_counter`: every block adds 1 (release) once its rows of the window have landed, so a GEMM that is already
// running can start on them.  `wait_counter`: the rows are still being written by a running GEMM; the kernel first
// waits (bounded) for ((rows of the window) / 256) * arrivals_per_row_block arrivals.
// `q_out` / `q_sc_out` (dispatch; 32-byte aligned rows, hidden % 128 == 0): the pulled (and scaled) rows also as E4M3
// [rows, hidden] with packed scales, quantised along the columns, addressed by schedule row like `dst`.
int comm_default_blocks();
int dispatch_rows_impl(const uint64_t* src_ptrs_host, int ep_size, const int32_t* peer_rank,
                       const int32_t* peer_token_idx, const int32_t* num_rows, int max_rows, int row_begin, int row_end,
                       int row_divisor, int64_t hidden, void* dst, const uint64_t* row_scale_ptrs_host,
                       float* row_scale_out, int blocks, cudaStream_t s, int32_t* done_counter = nullptr,
                       void* q_out = nullptr, void* q_sc_out = nullptr, int64_t index_limit = 0, int32_t* status = nullptr);
int combine_rows_impl(const void* src, const uint64_t* dst_ptrs_host, int ep_size, const int32_t* peer_rank,
                      const int32_t* peer_token_idx, const int32_t* num_rows, int max_rows, int row_begin, int row_end,
                      int64_t hidden, const float* row_values, const uint64_t* value_ptrs_host, int blocks, cudaStream_t s,
                      const int32_t* wait_counter = nullptr, int arrivals_per_row_block = 0, int32_t* status = nullptr,
                      int64_t index_limit = 0);

// MXFP8 codec launchers (quantize.cu).  Rows [row_begin, min(row_end, *num_rows)) are processed (row_end = 0: all
// M / rows_cap rows; `num_rows` is a device pointer, optional).  Row numbers are the caller's: a buffer holding only
// rows [first, first + M) is passed with every pointer moved back by `first` rows (transposed tensors: by `first`
// bytes, scale tensors: by first / 128 tiles along the row axis), and M / rows_cap stays the buffer's own row count,
// which is also the row stride of the transposed outputs.
// On `blocks` CTAs (0 = as many as there are tiles, up to 16 per SM); `done_counter`: every block of the launch adds 1
// (release) when it is through, so the window is quantised when the counter has grown by `blocks`.
int quantize_impl(const void* x_bf16, int64_t E, int64_t M, int64_t N, const int32_t* num_rows, int row_begin, int row_end,
                  void* x_fp8, void* x_sc, void* x_fp8_t, void* x_sc_t, cudaStream_t stream, int blocks = 0,
                  int32_t* done_counter = nullptr);
int swiglu_bwd_quant_impl(const void* gate_q, const void* gate_sc, const void* up_q, const void* up_sc, const void* d_hidden,
                          int64_t rows_cap, int64_t I, const int32_t* num_rows, int row_begin, int row_end, int has_limit, float limit,
                          const float* row_scale, void* dg_q, void* dg_sc, void* dg_qt, void* dg_sct,
                          void* du_q, void* du_sc, void* du_qt, void* du_sct, float* partials, float* row_grad,
                          cudaStream_t stream);

// ---------------------------------------------------------------- device side
#ifdef __CUDACC__

constexpr int kPeerMax = MOKB_MAX_EP;

struct PeerPtrs {               // by-value kernel argument: one base pointer per EP rank
    void* p[kPeerMax];
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ int lane_id() { return threadIdx.x & 31; }

__device__ __forceinline__ bool elect_one() {
    uint32_t pred = 0;
    asm volatile(
        "{\n"
        ".reg .pred P;\n"
        "elect.sync _|P, 0xffffffff;\n"
        "selp.u32 %0, 1, 0, P;\n"
        "}\n" : "=r"(pred));
    return pred != 0;
}

// ---- mbarrier
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_barrier_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async_smem() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n" : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}

// Every wait in this library is bounded.  A wait that runs out records `code`
// in the global status word, raises the CTA-wide abort flag and returns false;
// every other waiter of the CTA sees the flag within ~1k polls and returns
// false too, so the kernel drains and exits instead of hanging the GPU.
constexpr uint32_t kWaitFastPolls = 2048;
constexpr uint32_t kWaitLimit = 12u * 1000u * 1000u;   // x >=64 ns of back-off: roughly a second

__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                          int* status, int code) {
    for (uint32_t i = 0;; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if (i > kWaitFastPolls) __nanosleep(64);
        if ((i & 1023u) == 1023u) {
            if (*abort_flag) return false;
            if (i > kWaitLimit) {
                *abort_flag = 1;
                if (status) atomicCAS(status, 0, code);
                return false;
            }
        }
    }
}

// ---- counters between kernels (and between CTAs of one kernel): the producer of some rows adds to a global
// counter with release semantics after its stores, the consumer polls it with acquire loads.  The reference's
// barrier_wait / barrier_arrive (csrc/megakernel/utils.cuh:1-13) with a time limit: a consumer that waits longer
// than kFlagWaitNs records MOKB_ST_FLAG_TIMEOUT, raises the CTA's abort flag (if it has one) and gives up.
constexpr unsigned long long kFlagWaitNs = 2ull * 1000 * 1000 * 1000;

__device__ __forceinline__ int ld_acquire_gpu(const int* p) {
    int v;
    asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void red_release_gpu_add(int* p, int v) {
    asm volatile("red.release.gpu.global.add.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned long long global_timer_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
// makes writes that other threads made through ordinary stores (and that this thread has acquired) visible to
// the TMA reads this thread issues next
__device__ __forceinline__ void fence_proxy_async_global() { asm volatile("fence.proxy.async.global;" ::: "memory"); }

// `kind` / `index` say which counter it was (status words 1..3, for diagnosis: kind, index, value seen << 16 | target)
enum { kWaitWindowReady = 1, kWaitBlockDone = 2, kWaitWindowDone = 3 };

__device__ __forceinline__ bool flag_wait(const int* flag, int target, volatile int* abort_flag, int* status, int kind, int index) {
    unsigned long long t0 = 0;
    for (uint32_t i = 0;; ++i) {
        const int seen = ld_acquire_gpu(flag);
        if (seen >= target) return true;
        if (i >= 32) __nanosleep(i < 1024 ? 100 : 500);
        if ((i & 127u) == 127u) {
            if (abort_flag && *abort_flag) return false;
            const unsigned long long now = global_timer_ns();
            if (t0 == 0) t0 = now;
            if (now - t0 > kFlagWaitNs) {
                if (abort_flag) *abort_flag = 1;
                if (status && atomicCAS(status, 0, MOKB_ST_FLAG_TIMEOUT) == 0) {
                    status[1] = kind;
                    status[2] = index;
                    status[3] = (seen << 16) | (target & 0xFFFF);
                }
                return false;
            }
        }
    }
}

// Routes are numbered [0, limit) on every rank; an index outside (a stale or foreign schedule) must not become an access
// to a peer's memory: the row is skipped and the status words say where (limit <= 0: unchecked).
struct IndexGuard {
    int limit;
    int32_t* status;
};
enum { kBadIndexPull = 1, kBadIndexPush = 2, kBadIndexGemmPush = 3 };

__device__ __forceinline__ bool index_ok(const IndexGuard& g, int idx, int kind, int row) {
    if (g.limit <= 0 || (idx >= 0 && idx < g.limit)) return true;
    if (g.status && atomicCAS(g.status, 0, MOKB_ST_BAD_INDEX) == 0) {
        g.status[1] = kind;
        g.status[2] = row;
        g.status[3] = idx;
    }
    return false;
}

// ---- TMA
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* t) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(t)) : "memory");
}
__device__ __forceinline__ void tma_load_2d(uint32_t smem_dst, const CUtensorMap* t, uint32_t bar, int c0, int c1) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_dst), "l"(reinterpret_cast<uint64_t>(t)), "r"(bar), "r"(c0), "r"(c1) : "memory");
}

// ---- tcgen05 / TMEM
__device__ __forceinline__ void tmem_alloc(uint32_t smem_result, uint32_t ncols) {   // whole warp
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_result), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {                                  // whole warp
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {       // whole warp
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// D[tmem] (+)= A[smem desc] * B[smem desc], bf16 inputs, fp32 accumulate.
__device__ __forceinline__ void umma_bf16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n"
        "}\n" ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
// Block-scaled E4M3 x E4M3 with one E8M0 scale per 32 elements of K (scales in TMEM).
__device__ __forceinline__ void umma_mxf8(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                          uint32_t sfa_tmem, uint32_t sfb_tmem, uint32_t accumulate) {
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%5], [%6], p;\n"
        "}\n" ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(sfa_tmem), "r"(sfb_tmem) : "memory");
}
// smem -> TMEM copy of one 32x128b scale tile, replicated to the four 32-lane quarters.
__device__ __forceinline__ void tmem_cp_32x128b_warpx4(uint32_t taddr, uint64_t smem_desc) {
    asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(smem_desc) : "memory");
}

// ---- CTA pairs (cluster of 2, tcgen05 cta_group::2): the even CTA of the pair issues the MMAs,
// each CTA stages its own half of A and B, and barriers are signalled across the pair.
__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// address of the same shared-memory location in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t map_to_cta(uint32_t smem_addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
    return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// TMA load of this CTA's tile whose completion bytes are counted on a barrier of the pair's leader
// (every CTA fetches only the half-tiles it stages itself).
__device__ __forceinline__ void tma_load_2d_pair(uint32_t smem_dst, const CUtensorMap* t, uint32_t leader_bar, int c0, int c1) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_dst), "l"(reinterpret_cast<uint64_t>(t)), "r"(leader_bar), "r"(c0), "r"(c1) : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t smem_result, uint32_t ncols) {    // same warp in both CTAs
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_result), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// 256 x N x 16 MMA over the pair: rows 0..127 of A and D live in the leader, 128..255 in its peer,
// and each CTA holds half of the N columns of B.
__device__ __forceinline__ void umma_bf16_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n"
        "}\n" ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
// Block-scaled E4M3 MMA over the pair; scale bytes are picked by the a_sf_id / b_sf_id fields of `idesc`.
__device__ __forceinline__ void umma_mxf8_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                               uint32_t sfa_tmem, uint32_t sfb_tmem, uint32_t accumulate) {
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::2.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%5], [%6], p;\n"
        "}\n" ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(sfa_tmem), "r"(sfb_tmem) : "memory");
}
// smem -> TMEM copy of one 32 x 16-byte scale tile in both CTAs of the pair (each from its own smem),
// replicated to the four 32-lane quarters.
__device__ __forceinline__ void tmem_cp_32x128b_warpx4_pair(uint32_t taddr, uint64_t smem_desc) {
    asm volatile("tcgen05.cp.cta_group::2.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(smem_desc) : "memory");
}
// Shared-memory descriptor of an un-swizzled K-major tile whose rows are 16 bytes wide (a scale tile):
// 8-row groups 128 B apart.
__device__ __forceinline__ uint64_t make_smem_desc_plain16(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((smem_addr >> 4) & 0x3FFF);
    d |= static_cast<uint64_t>(1) << 16;           // LBO: one 16-byte unit (the tile is a single unit wide)
    d |= static_cast<uint64_t>(128 >> 4) << 32;    // SBO: 128 B between 8-row groups
    d |= static_cast<uint64_t>(1) << 46;
    return d;
}

// arrive on the barrier at this offset in every CTA of `cta_mask` once the MMAs issued so far retire
__device__ __forceinline__ void umma_commit_pair(uint32_t bar, uint16_t cta_mask) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(bar), "h"(cta_mask) : "memory");
}

// 32 lanes x 32 consecutive fp32 columns: lane i of the warp's TMEM quarter -> thread i.
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
// The same wait, tied to the registers of a load that was left in flight across other work: nothing that reads
// them can be scheduled above it.
__device__ __forceinline__ void tmem_ld_wait_for(uint32_t (&r)[32]) {
    asm volatile("tcgen05.wait::ld.sync.aligned;"
                 : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7]),
                   "+r"(r[8]), "+r"(r[9]), "+r"(r[10]), "+r"(r[11]), "+r"(r[12]), "+r"(r[13]), "+r"(r[14]), "+r"(r[15]),
                   "+r"(r[16]), "+r"(r[17]), "+r"(r[18]), "+r"(r[19]), "+r"(r[20]), "+r"(r[21]), "+r"(r[22]), "+r"(r[23]),
                   "+r"(r[24]), "+r"(r[25]), "+r"(r[26]), "+r"(r[27]), "+r"(r[28]), "+r"(r[29]), "+r"(r[30]), "+r"(r[31])
                 :: "memory");
}

// Shared-memory matrix descriptor (tcgen05), 128-byte swizzle.
//   K-major operand : rows at 128 B pitch, 8-row groups 1024 B apart (SBO); LBO unused.
//   MN-major operand: 64-element (128 B) runs along MN, 8 k-rows per 1024 B group (SBO),
//                     next 64 elements of MN `lbo_bytes` further (LBO).
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((smem_addr >> 4) & 0x3FFF);
    d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3FFF) << 16;
    d |= static_cast<uint64_t>((sbo_bytes >> 4) & 0x3FFF) << 32;
    d |= static_cast<uint64_t>(1) << 46;          // descriptor version of sm_100
    d |= static_cast<uint64_t>(2) << 61;          // SWIZZLE_128B
    return d;
}

// ---- small numeric helpers
__device__ __forceinline__ float bf16_round(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 t = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&t);
}
__device__ __forceinline__ float2 unpack_bf16(uint32_t v) {
    return __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&v));
}

#endif  // __CUDACC__
}  // namespace mokb
