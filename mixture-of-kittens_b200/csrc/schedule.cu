// Routing schedule builder.
//
// Produces exactly the schedule of the reference (csrc/scheduler.cuh:35-147):
// per-expert segments padded to 256 rows, and inside a segment the routes of
// the R source ranks interleaved round-robin, where the j-th route of a
// (rank, expert) pair is counted in the order in which a 1024-thread block
// strides over that rank's route list (thread index first, then iteration).
//
// The reference launches E_l*R blocks that each re-read one rank's whole route
// list twice.  Here every route is read twice in total:
//   view a rank's routes as a matrix [iteration][1024 threads]; the reference
//   order is column-major over that matrix.  A column is split into RC row
//   chunks, giving V = 1024*RC "virtual columns" in order.
//   1. count   : one thread per virtual column histograms its routes by local
//                expert in shared memory -> colcnt[r][e][v]; block sums go to
//                cnt[e][r] with integer atomics.
//   2. finalize: tokens_per_expert, segment bases, num_tokens, overflow check.
//   3. scan    : exclusive scan of colcnt[r][e][:] over v (one block per row).
//   4. place   : same walk as 1 with the counters started at the scanned
//                prefix, so each route knows its j and computes its row with
//                the closed form of scheduler.cuh:134-139.
#include "common.cuh"

namespace mokb {
namespace {

constexpr int kThreadsOrder = 1024;   // the reference's block size, which defines the order
constexpr int kPad = 256;             // expert segment padding

struct SchedParams {
    const int32_t* topk_all;  // [R, routes]
    int R, routes, E_l, C, rank;
    int RC;                   // row chunks per column
    int rows_per_chunk;       // ceil(ceil(routes/1024) / RC)
    int V;                    // 1024 * RC
    int32_t* cnt;             // [E_l, R]
    int32_t* base;            // [E_l + 1]
    int32_t* overflow;        // [1]
    int32_t* colcnt;          // [R, E_l, V]
    int32_t* peer_rank;
    int32_t* peer_token_idx;
    int32_t* num_tokens;
    int32_t* tokens_per_expert;
    int32_t* status;
};

template <bool PLACE>
__global__ void walk_kernel(SchedParams p) {
    extern __shared__ int32_t sm[];
    const int cpb = blockDim.x;
    int32_t* counters = sm;                         // [E_l][cpb]
    int32_t* cnt_s = counters + p.E_l * cpb;        // [E_l][R]   (PLACE)
    int32_t* base_s = cnt_s + p.E_l * p.R;          // [E_l]      (PLACE)
    const int r = blockIdx.y;
    const int v0 = blockIdx.x * cpb;
    const int t = threadIdx.x;
    const int v = v0 + t;
    const int first = p.rank * p.E_l;

    if (PLACE) {
        if (*p.overflow) return;
        for (int i = t; i < p.E_l * p.R; i += cpb) cnt_s[i] = p.cnt[i];
        for (int i = t; i < p.E_l; i += cpb) base_s[i] = p.base[i];
        for (int e = 0; e < p.E_l; ++e)
            counters[e * cpb + t] = p.colcnt[(static_cast<size_t>(r) * p.E_l + e) * p.V + v];
    } else {
        for (int e = 0; e < p.E_l; ++e) counters[e * cpb + t] = 0;
    }
    __syncthreads();

    const int32_t* routes = p.topk_all + static_cast<size_t>(r) * p.routes;
    const int c = v / p.RC, q = v - c * p.RC;
    const int row0 = q * p.rows_per_chunk;
    constexpr int U = 8;
    for (int s0 = 0; s0 < p.rows_per_chunk; s0 += U) {
        int idx[U], ex[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int s = s0 + u;
            const int i = (row0 + s) * kThreadsOrder + c;
            idx[u] = (s < p.rows_per_chunk && i < p.routes) ? i : -1;
            ex[u] = idx[u] >= 0 ? __ldg(routes + idx[u]) - first : -1;
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int e = ex[u];
            if (idx[u] >= 0 && e >= 0 && e < p.E_l) {
                const int j = counters[e * cpb + t]++;
                if (PLACE) {
                    int dst = base_s[e];
                    const int32_t* ce = cnt_s + e * p.R;
                    for (int rr = 0; rr < p.R; ++rr) {
                        const int n = ce[rr];
                        dst += min(n, j) + ((rr < r && n > j) ? 1 : 0);
                    }
                    p.peer_rank[dst] = r;
                    p.peer_token_idx[dst] = idx[u];
                }
            }
        }
    }
    if (PLACE) return;
    __syncthreads();
    for (int e = 0; e < p.E_l; ++e)
        p.colcnt[(static_cast<size_t>(r) * p.E_l + e) * p.V + v] = counters[e * cpb + t];
    // block total per expert -> cnt[e][r]
    const int warp = t >> 5, lane = t & 31, nwarps = cpb >> 5;
    for (int e = warp; e < p.E_l; e += nwarps) {
        int s = 0;
        for (int k = lane; k < cpb; k += 32) s += counters[e * cpb + k];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
        if (lane == 0 && s) atomicAdd(&p.cnt[e * p.R + r], s);
    }
}

__device__ __forceinline__ int block_exclusive_scan_1024(int x, int32_t* warp_sums, int* total) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    int inc = x;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const int n = __shfl_up_sync(0xffffffffu, inc, o);
        if (lane >= o) inc += n;
    }
    if (lane == 31) warp_sums[warp] = inc;
    __syncthreads();
    if (warp == 0) {
        int w = warp_sums[lane];
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int n = __shfl_up_sync(0xffffffffu, w, o);
            if (lane >= o) w += n;
        }
        warp_sums[lane] = w;
    }
    __syncthreads();
    const int before = warp ? warp_sums[warp - 1] : 0;
    if (total) *total = warp_sums[31];
    __syncthreads();
    return before + inc - x;
}

__global__ void finalize_kernel(SchedParams p) {
    __shared__ int32_t warp_sums[32];
    int carry = 0;
    for (int e0 = 0; e0 < p.E_l; e0 += 1024) {
        const int e = e0 + threadIdx.x;
        int padded = 0;
        if (e < p.E_l) {
            int n = 0;
            for (int r = 0; r < p.R; ++r) n += p.cnt[e * p.R + r];
            padded = (n + kPad - 1) / kPad * kPad;
            p.tokens_per_expert[e] = padded;
        }
        int total;
        const int ex = block_exclusive_scan_1024(padded, warp_sums, &total);
        if (e < p.E_l) p.base[e] = carry + ex;
        carry += total;
    }
    if (threadIdx.x == 0) {
        p.base[p.E_l] = carry;
        p.num_tokens[0] = carry;
        const int over = carry > p.C;
        *p.overflow = over;
        if (over) atomicCAS(p.status, MOKB_ST_OK, MOKB_ST_SCHEDULE_OVERFLOW);
    }
}

__global__ void scan_kernel(SchedParams p) {
    __shared__ int32_t warp_sums[32];
    int32_t* row = p.colcnt + static_cast<size_t>(blockIdx.x) * p.V;
    const int RC = p.RC;
    int local[8];
    int sum = 0;
    for (int k = 0; k < RC; ++k) { local[k] = row[threadIdx.x * RC + k]; sum += local[k]; }
    int run = block_exclusive_scan_1024(sum, warp_sums, nullptr);
    for (int k = 0; k < RC; ++k) { row[threadIdx.x * RC + k] = run; run += local[k]; }
}

}  // namespace
}  // namespace mokb

using namespace mokb;

static void sched_geometry(int R, int routes, int E_l, int* RC, int* rows_per_chunk, int* cpb) {
    const int P = (routes + kThreadsOrder - 1) / kThreadsOrder;
    int rc = 1;
    while (rc < 8 && R * kThreadsOrder * rc < 16384 && P / (rc * 2) >= 8) rc *= 2;
    *RC = rc;
    *rows_per_chunk = (P + rc - 1) / rc;
    int c = 128;
    while (c > 32 && static_cast<size_t>(E_l) * c * 4 > 160 * 1024) c /= 2;
    *cpb = c;
}

extern "C" size_t mokb_schedule_scratch_bytes(int ep_size, int num_local_experts) {
    const size_t E = static_cast<size_t>(ep_size) * num_local_experts;
    // cnt + base + overflow (rounded up), then colcnt at the largest RC
    size_t head = (E + num_local_experts + 2) * 4;
    head = (head + 255) / 256 * 256;
    return head + E * kThreadsOrder * 8 * 4;
}

extern "C" int mokb_schedule(const int32_t* topk_all, int ep_size, int num_local_tokens, int topk,
                             int num_local_experts, int schedule_capacity, int rank,
                             int32_t* peer_rank, int32_t* peer_token_idx, int32_t* num_tokens,
                             int32_t* tokens_per_expert, void* scratch, int32_t* status, void* stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    TraceScope trace(stream, "schedule");
    MOKB_REQUIRE(topk_all && peer_rank && peer_token_idx && num_tokens && tokens_per_expert && scratch && status,
                 "schedule: null pointer");
    MOKB_REQUIRE(ep_size >= 1 && ep_size <= MOKB_MAX_EP, "schedule: ep_size %d out of range", ep_size);
    MOKB_REQUIRE(rank >= 0 && rank < ep_size, "schedule: rank %d not in [0, %d)", rank, ep_size);
    MOKB_REQUIRE(num_local_tokens > 0 && topk > 0 && num_local_experts > 0, "schedule: sizes must be positive");
    MOKB_REQUIRE(schedule_capacity > 0 && schedule_capacity % kPad == 0, "schedule: capacity must be a positive multiple of 256");
    const long long routes_ll = 1LL * num_local_tokens * topk;
    MOKB_REQUIRE(routes_ll * ep_size < (1LL << 31), "schedule: too many routes");
    MOKB_REQUIRE(static_cast<size_t>(num_local_experts) * 32 * 4 <= 160 * 1024, "schedule: too many local experts");

    SchedParams p;
    p.topk_all = topk_all;
    p.R = ep_size; p.routes = static_cast<int>(routes_ll); p.E_l = num_local_experts;
    p.C = schedule_capacity; p.rank = rank;
    int cpb;
    sched_geometry(p.R, p.routes, p.E_l, &p.RC, &p.rows_per_chunk, &cpb);
    p.V = kThreadsOrder * p.RC;
    const size_t E = static_cast<size_t>(p.R) * p.E_l;
    int32_t* s = static_cast<int32_t*>(scratch);
    p.cnt = s;
    p.base = s + E;
    p.overflow = p.base + p.E_l + 1;
    size_t head = (E + p.E_l + 2) * 4;
    head = (head + 255) / 256 * 256;
    p.colcnt = reinterpret_cast<int32_t*>(static_cast<char*>(scratch) + head);
    p.peer_rank = peer_rank; p.peer_token_idx = peer_token_idx;
    p.num_tokens = num_tokens; p.tokens_per_expert = tokens_per_expert; p.status = status;

    MOKB_CUDA(cudaMemsetAsync(p.cnt, 0, head, stream));
    MOKB_CUDA(cudaMemsetAsync(peer_rank, 0xFF, static_cast<size_t>(schedule_capacity) * 4, stream));
    MOKB_CUDA(cudaMemsetAsync(peer_token_idx, 0xFF, static_cast<size_t>(schedule_capacity) * 4, stream));

    const size_t smem = (static_cast<size_t>(p.E_l) * cpb + E + p.E_l) * 4;
    MOKB_CUDA(cudaFuncSetAttribute(walk_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    MOKB_CUDA(cudaFuncSetAttribute(walk_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    const dim3 grid(p.V / cpb, p.R);
    walk_kernel<false><<<grid, cpb, smem, stream>>>(p);
    finalize_kernel<<<1, 1024, 0, stream>>>(p);
    scan_kernel<<<static_cast<unsigned>(E), 1024, 0, stream>>>(p);
    walk_kernel<true><<<grid, cpb, smem, stream>>>(p);
    MOKB_CUDA(cudaGetLastError());
    note_launch(4);
    return MOKB_OK;
}

// ---------------------------------------------------------------------------
// Routing schedule for callers that must not allocate device memory.
//
// Some hosts of this library run where cudaMalloc is off limits: inside a
// framework that owns the whole device heap through its own pool, in a
// latency-critical step loop where an allocation would serialise the device,
// or in a process that pre-commits all memory at start-up.  For them the work
// area of the schedule builder lives in the library image itself: a fixed
// __device__ array that every GPU loading the library carries until exit.
// The price is a size limit and shared state (see the header).
namespace mokb {
namespace {

constexpr size_t kStaticHeadBytes = 16u << 10;     // cnt[E] + base[E_l + 1] + overflow flag
constexpr size_t kStaticColcntBytes = 4u << 20;    // colcnt[E][1024 * RC]: E * RC <= 1024
static __device__ __align__(256) unsigned char g_static_sched_scratch[kStaticHeadBytes + kStaticColcntBytes];

// Device address of the array above, per device.  In host code the array's name is only a
// handle for the runtime; the address a kernel can use comes from cudaGetSymbolAddress,
// asked for with that device current.
void* g_static_sched_ptr[64] = {nullptr};

int static_sched_scratch(void** out) {
    int dev = -1;
    MOKB_CUDA(cudaGetDevice(&dev));
    MOKB_REQUIRE(dev >= 0 && dev < 64, "schedule_noalloc: device index %d out of range", dev);
    if (g_static_sched_ptr[dev] == nullptr) {
        void* p = nullptr;
        MOKB_CUDA(cudaGetSymbolAddress(&p, g_static_sched_scratch));
        MOKB_REQUIRE(p != nullptr, "schedule_noalloc: cudaGetSymbolAddress returned a null address");
        g_static_sched_ptr[dev] = p;
    }
    *out = g_static_sched_ptr[dev];
    return MOKB_OK;
}

}  // namespace
}  // namespace mokb

extern "C" int mokb_schedule_noalloc(const int32_t* topk_all, int ep_size, int num_local_tokens, int topk,
                                     int num_local_experts, int schedule_capacity, int rank,
                                     int32_t* peer_rank, int32_t* peer_token_idx, int32_t* num_tokens,
                                     int32_t* tokens_per_expert, int32_t* status, void* stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    MOKB_REQUIRE(topk_all && peer_rank && peer_token_idx && num_tokens && tokens_per_expert && status,
                 "schedule_noalloc: null pointer");
    MOKB_REQUIRE(ep_size >= 1 && ep_size <= MOKB_MAX_EP, "schedule_noalloc: ep_size %d out of range", ep_size);
    MOKB_REQUIRE(rank >= 0 && rank < ep_size, "schedule_noalloc: rank %d not in [0, %d)", rank, ep_size);
    MOKB_REQUIRE(num_local_tokens > 0 && topk > 0 && num_local_experts > 0, "schedule_noalloc: sizes must be positive");
    MOKB_REQUIRE(schedule_capacity > 0 && schedule_capacity % kPad == 0,
                 "schedule_noalloc: capacity must be a positive multiple of 256");
    const long long routes_ll = 1LL * num_local_tokens * topk;
    MOKB_REQUIRE(routes_ll * ep_size < (1LL << 31), "schedule_noalloc: too many routes");
    const size_t E = static_cast<size_t>(ep_size) * num_local_experts;
    MOKB_REQUIRE(E <= MOKB_SCHEDULE_NOALLOC_MAX_EXPERTS,
                 "schedule_noalloc: ep_size * num_local_experts = %zu exceeds the built-in work area's limit of %d experts; "
                 "use mokb_schedule with caller-provided scratch", E, MOKB_SCHEDULE_NOALLOC_MAX_EXPERTS);
    MOKB_REQUIRE(static_cast<size_t>(num_local_experts) * 32 * 4 <= 160 * 1024, "schedule_noalloc: too many local experts");

    void* scratch = nullptr;
    MOKB_TRY(static_sched_scratch(&scratch));

    SchedParams p;
    p.topk_all = topk_all;
    p.R = ep_size; p.routes = static_cast<int>(routes_ll); p.E_l = num_local_experts;
    p.C = schedule_capacity; p.rank = rank;
    int cpb;
    sched_geometry(p.R, p.routes, p.E_l, &p.RC, &p.rows_per_chunk, &cpb);
    // fewer row chunks per column until colcnt fits the fixed area (the result does not depend on RC)
    while (p.RC > 1 && E * kThreadsOrder * p.RC * 4 > kStaticColcntBytes) p.RC /= 2;
    const int P = (p.routes + kThreadsOrder - 1) / kThreadsOrder;
    p.rows_per_chunk = (P + p.RC - 1) / p.RC;
    p.V = kThreadsOrder * p.RC;
    MOKB_REQUIRE(E * p.V * 4 <= kStaticColcntBytes && (E + p.E_l + 2) * 4 <= kStaticHeadBytes,
                 "schedule_noalloc: problem does not fit the built-in work area");
    int32_t* s = static_cast<int32_t*>(scratch);
    p.cnt = s;
    p.base = s + E;
    p.overflow = p.base + p.E_l + 1;
    p.colcnt = reinterpret_cast<int32_t*>(static_cast<char*>(scratch) + kStaticHeadBytes);
    p.peer_rank = peer_rank; p.peer_token_idx = peer_token_idx;
    p.num_tokens = num_tokens; p.tokens_per_expert = tokens_per_expert; p.status = status;

    // the area keeps whatever the previous call left: the counters and the overflow flag must start at zero
    // (colcnt is fully rewritten by the counting pass before anything reads it)
    MOKB_CUDA(cudaMemsetAsync(scratch, 0, kStaticHeadBytes, stream));
    MOKB_CUDA(cudaMemsetAsync(peer_rank, 0xFF, static_cast<size_t>(schedule_capacity) * 4, stream));
    MOKB_CUDA(cudaMemsetAsync(peer_token_idx, 0xFF, static_cast<size_t>(schedule_capacity) * 4, stream));

    const size_t smem = (static_cast<size_t>(p.E_l) * cpb + E + p.E_l) * 4;
    MOKB_CUDA(cudaFuncSetAttribute(walk_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    MOKB_CUDA(cudaFuncSetAttribute(walk_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    const dim3 grid(p.V / cpb, p.R);
    walk_kernel<false><<<grid, cpb, smem, stream>>>(p);
    finalize_kernel<<<1, 1024, 0, stream>>>(p);
    scan_kernel<<<static_cast<unsigned>(E), 1024, 0, stream>>>(p);
    walk_kernel<true><<<grid, cpb, smem, stream>>>(p);
    MOKB_CUDA(cudaGetLastError());
    note_launch(4);
    return MOKB_OK;
}
