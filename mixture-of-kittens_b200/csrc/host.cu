// Host-side plumbing shared by every entry point: thread-local error text,
// device queries, and TMA tensor-map encoding through the driver entry point
// (looked up at run time, so the library links against the CUDA runtime only
// and still loads on a machine without a driver).
#include <stdarg.h>
#include <string.h>

#include "common.cuh"

namespace mokb {

static thread_local char g_error[512] = "";
static unsigned long long g_launches = 0;

void note_launch(int n) { __atomic_fetch_add(&g_launches, (unsigned long long)n, __ATOMIC_RELAXED); }

void set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, ap);
    va_end(ap);
}

int cuda_fail(cudaError_t e, const char* what, const char* file, int line) {
    set_error("CUDA error %d (%s) at %s:%d in %s", (int)e, cudaGetErrorString(e), file, line, what);
    return MOKB_ERR_CUDA;
}

int sm_count() {
    static int cached[64] = {0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    if (cached[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        cached[dev] = n;
    }
    return cached[dev];
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    }
    return fn;
}

int make_tmap_2d(CUtensorMap* out, const void* base, int elem_bytes, uint64_t inner, uint64_t outer,
                 uint64_t row_stride_bytes, uint32_t box_inner, uint32_t box_outer) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) {
        set_error("cuTensorMapEncodeTiled is not available (no CUDA driver?)");
        return MOKB_ERR_CUDA;
    }
    MOKB_REQUIRE((reinterpret_cast<uintptr_t>(base) & 15) == 0, "tensor base %p is not 16-byte aligned", base);
    MOKB_REQUIRE(row_stride_bytes % 16 == 0, "row stride %llu B is not a multiple of 16", (unsigned long long)row_stride_bytes);
    // elem_bytes 2 = bf16 and 1 = u8, 128-byte swizzle; elem_bytes 4 = u32 rows copied as they are (scale tiles)
    const bool plain = elem_bytes == 4;
    MOKB_REQUIRE(plain || box_inner * elem_bytes == 128, "swizzled box must be 128 B wide");
    MOKB_REQUIRE(box_inner <= 256 && box_outer >= 1 && box_outer <= 256, "box %ux%u out of range", box_inner, box_outer);
    cuuint64_t dims[2] = {inner, outer};
    cuuint64_t strides[1] = {row_stride_bytes};
    cuuint32_t box[2] = {box_inner, box_outer};
    cuuint32_t estr[2] = {1, 1};
    CUtensorMapDataType dt = elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                             : elem_bytes == 4 ? CU_TENSOR_MAP_DATA_TYPE_UINT32 : CU_TENSOR_MAP_DATA_TYPE_UINT8;
    CUresult r = fn(out, dt, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    plain ? CU_TENSOR_MAP_SWIZZLE_NONE : CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        set_error("cuTensorMapEncodeTiled failed with CUresult %d (inner=%llu outer=%llu stride=%llu box=%ux%u)", (int)r,
                  (unsigned long long)inner, (unsigned long long)outer, (unsigned long long)row_stride_bytes, box_inner, box_outer);
        return MOKB_ERR_CUDA;
    }
    return MOKB_OK;
}

}  // namespace mokb

extern "C" const char* mokb_last_error(void) { return mokb::g_error; }

extern "C" int mokb_sm_count(void) { return mokb::sm_count(); }

// ---------------------------------------------------------------- launch timeline
namespace mokb {
namespace {
struct TraceRec {
    cudaEvent_t begin, end;
    const char* tag;
    int arg;
    cudaStream_t stream;
};
constexpr int kTraceMax = 8192;
TraceRec g_trace[kTraceMax];
int g_trace_n = 0;
bool g_trace_on = false;
cudaEvent_t g_trace_t0 = nullptr;
}  // namespace

TraceScope::TraceScope(cudaStream_t stream, const char* tag, int arg) : slot_(-1), stream_(stream) {
    if (!g_trace_on || g_trace_n >= kTraceMax) return;
    TraceRec& r = g_trace[g_trace_n];
    if (!r.begin && (cudaEventCreate(&r.begin) != cudaSuccess || cudaEventCreate(&r.end) != cudaSuccess)) return;
    r.tag = tag;
    r.arg = arg;
    r.stream = stream;
    if (cudaEventRecord(r.begin, stream) != cudaSuccess) return;
    slot_ = g_trace_n++;
}
TraceScope::~TraceScope() {
    if (slot_ >= 0) cudaEventRecord(g_trace[slot_].end, stream_);
}
}  // namespace mokb

extern "C" int mokb_trace_begin(void* stream) {
    using namespace mokb;
    if (!g_trace_t0) MOKB_CUDA(cudaEventCreate(&g_trace_t0));
    g_trace_n = 0;
    MOKB_CUDA(cudaEventRecord(g_trace_t0, static_cast<cudaStream_t>(stream)));
    g_trace_on = true;
    return MOKB_OK;
}

extern "C" long long mokb_trace_end(char* out, size_t cap) {
    using namespace mokb;
    g_trace_on = false;
    if (cudaDeviceSynchronize() != cudaSuccess) return -1;
    // streams are numbered in order of first appearance
    cudaStream_t seen[16];
    int n_seen = 0;
    size_t used = 0;
    for (int i = 0; i < g_trace_n; ++i) {
        const TraceRec& r = g_trace[i];
        int sid = 0;
        while (sid < n_seen && seen[sid] != r.stream) ++sid;
        if (sid == n_seen && n_seen < 16) seen[n_seen++] = r.stream;
        float t0 = 0.f, t1 = 0.f;
        if (cudaEventElapsedTime(&t0, g_trace_t0, r.begin) != cudaSuccess || cudaEventElapsedTime(&t1, g_trace_t0, r.end) != cudaSuccess)
            continue;
        char line[160];
        const int len = snprintf(line, sizeof(line), "%s %d %d %.4f %.4f\n", r.tag, r.arg, sid, t0, t1);
        if (out && used + len < cap) memcpy(out + used, line, len);
        used += len;
    }
    if (out && cap) out[used < cap ? used : cap - 1] = 0;
    g_trace_n = 0;
    return static_cast<long long>(used);
}

extern "C" unsigned long long mokb_launch_count(void) { return __atomic_load_n(&mokb::g_launches, __ATOMIC_RELAXED); }

extern "C" int mokb_device_arch(void) {
    int dev = 0, major = 0, minor = 0;
    MOKB_CUDA(cudaGetDevice(&dev));
    MOKB_CUDA(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev));
    MOKB_CUDA(cudaDeviceGetAttribute(&minor, cudaDevAttrComputeCapabilityMinor, dev));
    return major * 10 + minor;
}

// sizeof() of the argument structs, so a foreign-language binding can check its own layout.
extern "C" int mokb_struct_sizes(int* out, int n) {
    const int sizes[3] = {(int)sizeof(mokb_fwd_bf16_args), (int)sizeof(mokb_bwd_bf16_args), (int)sizeof(mokb_gemm_args)};
    for (int i = 0; i < n && i < 3; ++i) out[i] = sizes[i];
    return 3;
}

extern "C" int mokb_struct_sizes_mxfp8(int* out, int n) {
    const int sizes[3] = {(int)sizeof(mokb_fwd_mxfp8_args), (int)sizeof(mokb_bwd_mxfp8_args), (int)sizeof(mokb_gemm_fp8_args)};
    for (int i = 0; i < n && i < 3; ++i) out[i] = sizes[i];
    return 3;
}
