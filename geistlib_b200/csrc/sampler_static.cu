/*
 * sampler_static.cu — greedy argmax over a batch of rows that allocates nothing.
 *
 * Who needs it. Every other entry point takes a context whose scratch comes from
 * cudaMalloc, and the context grows that scratch when a larger batch arrives. Some
 * callers cannot afford that: an engine that hands the whole device to its own arena
 * at start-up and leaves no room for a late cudaMalloc; a decode loop that promised
 * its user a fixed memory footprint per token (the reference's sampler makes that
 * promise for its hot path, src/engine/sampler.c:9-11 of geistlib); a serving thread
 * that must not take the driver's allocation lock, which serialises against every
 * other stream of the process and can stall for milliseconds. For them the scratch
 * lives in the image of this library: a file-scope __device__ array whose address is
 * looked up once per device and handed to the kernel as a plain pointer.
 *
 * The kernel is the greedy mode of the streaming sampler reduced to its two steps:
 * every CTA scans one slice of one row and leaves (max, first id) in the scratch; the
 * CTA that arrives last for a row folds the row's slices and writes the id. Ties go
 * to the lowest id and a row of -inf returns 0, as sampler.c:52-62 does.
 *
 * The scratch is shared by every call on a device: two calls that overlap in time (two
 * streams, two threads) race on it. The per-row arrival counters must be zero when the
 * kernel starts; the launcher clears them on the caller's stream before each launch.
 */
#include <cuda_runtime.h>
#include <math_constants.h>

#include <mutex>

#include "sampler_device.cuh"

namespace gb {

constexpr int kStaticSlice    = 8192;   /* floats one CTA scans: 256 threads x 8 float4 */
constexpr int kStaticThreads  = 256;
constexpr int kStaticMaxRows  = 4096;   /* rows per call */
constexpr int kStaticMaxItems = 65536;  /* rows x slices per call */
constexpr int kStaticMaxDev   = 64;

struct StaticScratch {
    int  arrived[kStaticMaxRows];   /* slices of a row that have been written; zero at launch */
    Pair partial[kStaticMaxItems];  /* (max, first id) of each slice */
};

/* 16 KB of counters + 512 KB of slice results */
static __device__ __align__(256) unsigned char g_static_scratch[sizeof(StaticScratch)];

__global__ void __launch_bounds__(kStaticThreads) argmax_rows_static_kernel(const float *__restrict__ logits, long long row_stride, int V, int n_slices,
                                                                            int aligned, StaticScratch *scratch, int *__restrict__ out) {
    __shared__ float s_v[kStaticThreads / 32];
    __shared__ int   s_a[kStaticThreads / 32];
    __shared__ int   s_last;

    const int    row  = blockIdx.x / n_slices;
    const int    s    = blockIdx.x - row * n_slices;
    const int    base = s * kStaticSlice;
    const int    n    = min(kStaticSlice, V - base);
    const float *p    = logits + (long long) row * row_stride + base;
    const int    tid  = threadIdx.x;

    float v = -CUDART_INF_F;
    int   a = 0x7fffffff;
    if (aligned) {
        const float4 *p4 = reinterpret_cast<const float4 *>(p);
        const int     n4 = n >> 2;
        float4        r[8];
#pragma unroll
        for (int i = 0; i < 8; i++) {
            const int j = tid + kStaticThreads * i;
            r[i] = j < n4 ? __ldcs(p4 + j) : make_float4(-CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F);
        }
#pragma unroll
        for (int i = 0; i < 8; i++) {
            const int j = tid + kStaticThreads * i;
            if (j < n4) {
                const int   id = base + 4 * j;
                const float x[4] = {r[i].x, r[i].y, r[i].z, r[i].w};
#pragma unroll
                for (int c = 0; c < 4; c++) { /* ids grow along the scan: strict > keeps the first */
                    if (x[c] > v || (x[c] == v && id + c < a)) {
                        v = x[c];
                        a = id + c;
                    }
                }
            }
        }
        for (int j = 4 * n4 + tid; j < n; j += kStaticThreads) { /* at most three trailing floats */
            const float x = p[j];
            if (x > v || (x == v && base + j < a)) {
                v = x;
                a = base + j;
            }
        }
    } else {
        for (int j = tid; j < n; j += kStaticThreads) {
            const float x = p[j];
            if (x > v || (x == v && base + j < a)) {
                v = x;
                a = base + j;
            }
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, v, o);
        const int   oa = __shfl_xor_sync(0xffffffffu, a, o);
        if (pair_before(ov, oa, v, a)) {
            v = ov;
            a = oa;
        }
    }
    if ((tid & 31) == 0) {
        s_v[tid >> 5] = v;
        s_a[tid >> 5] = a;
    }
    __syncthreads();
    if (tid == 0) {
        for (int w = 1; w < kStaticThreads / 32; w++) {
            if (pair_before(s_v[w], s_a[w], v, a)) {
                v = s_v[w];
                a = s_a[w];
            }
        }
        Pair r;
        r.v   = v;
        r.idx = a;
        scratch->partial[blockIdx.x] = r;
        __threadfence(); /* the slice result is visible before the arrival is counted */
        s_last = atomicAdd(&scratch->arrived[row], 1) == n_slices - 1;
    }
    __syncthreads();
    if (!s_last || tid >= 32) {
        return;
    }
    __threadfence(); /* order the reads below after the last arrival */
    v = -CUDART_INF_F;
    a = 0x7fffffff;
    for (int j = tid; j < n_slices; j += 32) {
        const Pair *q  = &scratch->partial[row * n_slices + j];
        const float qv = __ldcg(&q->v);
        const int   qa = __ldcg(&q->idx);
        if (pair_before(qv, qa, v, a)) {
            v = qv;
            a = qa;
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, v, o);
        const int   oa = __shfl_xor_sync(0xffffffffu, a, o);
        if (pair_before(ov, oa, v, a)) {
            v = ov;
            a = oa;
        }
    }
    if (tid == 0) {
        out[row] = a == 0x7fffffff ? 0 : a; /* a row of NaN keeps index 0 */
    }
}

int argmax_rows_static_max_rows(long long n_vocab) {
    if (n_vocab <= 0) {
        return 0;
    }
    const long long slices = (n_vocab + kStaticSlice - 1) / kStaticSlice;
    const long long rows   = kStaticMaxItems / slices;
    return (int) (rows < kStaticMaxRows ? rows : kStaticMaxRows);
}

/*
 * Looks the scratch address up on first use of a device (with that device current) and
 * launches. Returns cudaSuccess or the failing call's code; *what names the call.
 * Nothing here allocates device memory: cudaGetSymbolAddress only returns where the
 * module's own image already placed the array. The address is looked up once per device and
 * kept for the life of the process: after cudaDeviceReset (or any other teardown of the
 * device's primary context) it is stale and this entry must not be called again.
 */
cudaError_t launch_argmax_rows_static(int device, const float *logits, long long row_stride, int n_rows, int V, int *out, cudaStream_t stream, const char **what) {
    static std::mutex     mu;
    static StaticScratch *addr[kStaticMaxDev] = {};
    *what = "";
    if (device < 0 || device >= kStaticMaxDev) {
        *what = "device index";
        return cudaErrorInvalidDevice;
    }
    /* the caller's current device is put back on every way out */
    struct DeviceGuard {
        int prev = -1;
        ~DeviceGuard() {
            if (prev >= 0) {
                cudaSetDevice(prev);
            }
        }
    } guard;
    int         cur = -1;
    cudaError_t e   = cudaGetDevice(&cur);
    if (e != cudaSuccess) {
        *what = "cudaGetDevice";
        return e;
    }
    if (cur != device) {
        e = cudaSetDevice(device);
        if (e != cudaSuccess) {
            *what = "cudaSetDevice";
            return e;
        }
        guard.prev = cur;
    }
    StaticScratch *scratch;
    {
        std::lock_guard<std::mutex> lk(mu);
        if (addr[device] == nullptr) {
            void *ptr = nullptr;
            e = cudaGetSymbolAddress(&ptr, g_static_scratch);
            if (e != cudaSuccess) {
                *what = "cudaGetSymbolAddress";
                return e;
            }
            addr[device] = static_cast<StaticScratch *>(ptr);
        }
        scratch = addr[device];
    }
    const int n_slices = (V + kStaticSlice - 1) / kStaticSlice;
    e = cudaMemsetAsync(scratch->arrived, 0, sizeof(int) * (size_t) n_rows, stream);
    if (e != cudaSuccess) {
        *what = "cudaMemsetAsync";
        return e;
    }
    const int aligned = (reinterpret_cast<uintptr_t>(logits) % 16 == 0) && (row_stride % 4 == 0);
    argmax_rows_static_kernel<<<n_rows * n_slices, kStaticThreads, 0, stream>>>(logits, row_stride, V, n_slices, aligned, scratch, out);
    e = cudaGetLastError();
    if (e != cudaSuccess) {
        *what = "kernel launch";
    }
    return e;
}

} /* namespace gb */
