// Library-level entry points: version, errors, host-side corpus preparation,
// raw buffers.  The trainer lives in fv_train.cu, the hasher in fv_hash.cu.
#include <omp.h>

#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <string>
#include <vector>

#include "fv_common.h"

namespace fv {

static thread_local std::string g_last_error;

int fail(int code, const char* fmt, ...) {
  char buf[1024];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof(buf), fmt, ap);
  va_end(ap);
  g_last_error = buf;
  return code;
}

void clear_error() { g_last_error.clear(); }

}  // namespace fv

extern "C" {

int fv_version(void) { return FV_ABI_VERSION; }

const char* fv_last_error(void) { return fv::g_last_error.c_str(); }

int fv_device_count(int* count) {
  FV_REQUIRE(count != nullptr, FV_ERR_INVALID, "fv_device_count: count is NULL");
  *count = 0;
  FV_CUDA(cudaGetDeviceCount(count));
  return FV_OK;
}

// Window enumeration.  A chunk of `len` tokens contributes len-window+1 windows
// when window <= len < maxlen.  Window starts are counted from the running sum
// of chunk lengths (equal to offsets[s] when offsets[0] == 0).
int fv_enumerate_windows(const uint64_t* offsets, uint64_t nchunks, uint32_t window, uint32_t maxlen,
                         uint64_t* count, uint64_t* starts) {
  FV_REQUIRE(count != nullptr, FV_ERR_INVALID, "fv_enumerate_windows: count is NULL");
  FV_REQUIRE(window >= 1, FV_ERR_INVALID, "fv_enumerate_windows: window must be >= 1");
  *count = 0;
  if (nchunks == 0) return FV_OK;
  FV_REQUIRE(offsets != nullptr, FV_ERR_INVALID, "fv_enumerate_windows: offsets is NULL");
  if (maxlen == 0) maxlen = 214;
  for (uint64_t s = 0; s < nchunks; ++s)
    FV_REQUIRE(offsets[s + 1] >= offsets[s], FV_ERR_DATA,
               "fv_enumerate_windows: offsets decrease at chunk %llu", (unsigned long long)s);

  // Pass 1: windows per block of chunks; pass 2: fill, each block from its own base.
  const int nthreads = omp_get_max_threads();
  const uint64_t nblocks = (uint64_t)nthreads * 8;
  const uint64_t per = (nchunks + nblocks - 1) / nblocks;
  std::vector<uint64_t> block_windows(nblocks + 1, 0);
#pragma omp parallel for schedule(static)
  for (int64_t b = 0; b < (int64_t)nblocks; ++b) {
    uint64_t lo = (uint64_t)b * per, hi = lo + per < nchunks ? lo + per : nchunks;
    uint64_t c = 0;
    for (uint64_t s = lo; s < hi; ++s) {
      uint64_t len = offsets[s + 1] - offsets[s];
      if (len >= window && len < maxlen) c += len - window + 1;
    }
    block_windows[b + 1] = c;
  }
  for (uint64_t b = 0; b < nblocks; ++b) block_windows[b + 1] += block_windows[b];
  *count = block_windows[nblocks];
  if (starts == nullptr) return FV_OK;

  const uint64_t origin = offsets[0];
#pragma omp parallel for schedule(static)
  for (int64_t b = 0; b < (int64_t)nblocks; ++b) {
    uint64_t lo = (uint64_t)b * per, hi = lo + per < nchunks ? lo + per : nchunks;
    uint64_t out = block_windows[b];
    for (uint64_t s = lo; s < hi; ++s) {
      uint64_t len = offsets[s + 1] - offsets[s];
      if (len >= window && len < maxlen) {
        uint64_t first = offsets[s] - origin;  // running sum of the lengths before chunk s
        for (uint64_t i = 0; i + window <= len; ++i) starts[out++] = first + i;
      }
    }
  }
  return FV_OK;
}

int fv_inverse_frequency(const int32_t* enc, uint64_t ntok, uint32_t vocab, int saturate, float* inv_freq) {
  FV_REQUIRE(inv_freq != nullptr && vocab > 0, FV_ERR_INVALID, "fv_inverse_frequency: bad arguments");
  FV_REQUIRE(enc != nullptr || ntok == 0, FV_ERR_INVALID, "fv_inverse_frequency: enc is NULL");
  std::vector<uint64_t> counts(vocab, 0);
  int bad = 0;
#pragma omp parallel
  {
    std::vector<uint64_t> local(vocab, 0);
    int local_bad = 0;
#pragma omp for schedule(static) nowait
    for (int64_t i = 0; i < (int64_t)ntok; ++i) {
      int32_t t = enc[i];
      if (t < 0) continue;
      if ((uint32_t)t >= vocab) {
        local_bad = 1;
        continue;
      }
      local[t] += 1;
    }
#pragma omp critical
    {
      for (uint32_t v = 0; v < vocab; ++v) counts[v] += local[v];
      bad |= local_bad;
    }
  }
  FV_REQUIRE(!bad, FV_ERR_DATA, "fv_inverse_frequency: a token id is >= vocab (%u)", vocab);
  for (uint32_t v = 0; v < vocab; ++v) {
    uint64_t c = counts[v];
    if (saturate && c > (1ull << 24)) c = 1ull << 24;  // a float counter stops growing here
    inv_freq[v] = c ? (float)(1.0 / (double)c) : 0.0f;
  }
  return FV_OK;
}

int fv_shard_range(uint64_t num_windows, uint32_t batch, int32_t world, int32_t rank, uint64_t step,
                   uint64_t* first, uint64_t* count) {
  FV_REQUIRE(first && count, FV_ERR_INVALID, "fv_shard_range: output pointer is NULL");
  FV_REQUIRE(batch > 0 && world > 0 && rank >= 0 && rank < world, FV_ERR_INVALID,
             "fv_shard_range: need batch > 0 and 0 <= rank < world");
  // Global step `step` covers [step*world*batch, (step+1)*world*batch) of the
  // current order; rank g takes the g-th block of `batch`, clipped to the end.
  unsigned __int128 lo = (unsigned __int128)step * world * batch + (unsigned __int128)rank * batch;
  if (lo > num_windows) lo = num_windows;
  unsigned __int128 hi = lo + batch;
  if (hi > num_windows) hi = num_windows;
  *first = (uint64_t)lo;
  *count = (uint64_t)(hi - lo);
  return FV_OK;
}

int fv_device_alloc(int device, size_t bytes, void** ptr) {
  FV_REQUIRE(ptr != nullptr, FV_ERR_INVALID, "fv_device_alloc: ptr is NULL");
  fv::DeviceGuard g(device);
  FV_REQUIRE(g.ok, FV_ERR_CUDA, "fv_device_alloc: cannot select device %d", device);
  FV_CUDA(cudaMalloc(ptr, bytes ? bytes : 1));
  return FV_OK;
}

int fv_device_free(int device, void* ptr) {
  fv::DeviceGuard g(device);
  FV_REQUIRE(g.ok, FV_ERR_CUDA, "fv_device_free: cannot select device %d", device);
  FV_CUDA(cudaFree(ptr));
  return FV_OK;
}

int fv_host_alloc_pinned(size_t bytes, void** ptr) {
  FV_REQUIRE(ptr != nullptr, FV_ERR_INVALID, "fv_host_alloc_pinned: ptr is NULL");
  FV_CUDA(cudaHostAlloc(ptr, bytes ? bytes : 1, cudaHostAllocPortable));
  return FV_OK;
}

int fv_host_free_pinned(void* ptr) {
  FV_CUDA(cudaFreeHost(ptr));
  return FV_OK;
}

int fv_device_mem_info(int device, size_t* free_bytes, size_t* total_bytes) {
  FV_REQUIRE(free_bytes && total_bytes, FV_ERR_INVALID, "fv_device_mem_info: output pointer is NULL");
  fv::DeviceGuard g(device);
  FV_REQUIRE(g.ok, FV_ERR_CUDA, "fv_device_mem_info: cannot select device %d", device);
  FV_CUDA(cudaMemGetInfo(free_bytes, total_bytes));
  return FV_OK;
}

int fv_copy_to_device(int device, void* dst, const void* src, size_t bytes) {
  fv::DeviceGuard g(device);
  FV_REQUIRE(g.ok, FV_ERR_CUDA, "fv_copy_to_device: cannot select device %d", device);
  FV_CUDA(cudaMemcpy(dst, src, bytes, cudaMemcpyHostToDevice));
  return FV_OK;
}

int fv_copy_to_host(int device, void* dst, const void* src, size_t bytes) {
  fv::DeviceGuard g(device);
  FV_REQUIRE(g.ok, FV_ERR_CUDA, "fv_copy_to_host: cannot select device %d", device);
  FV_CUDA(cudaMemcpy(dst, src, bytes, cudaMemcpyDeviceToHost));
  return FV_OK;
}

}  // extern "C"

namespace {
__global__ void k_flush(uint4* buf, size_t n, uint32_t v) {
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  size_t stride = (size_t)gridDim.x * blockDim.x;
  for (; i < n; i += stride) buf[i] = make_uint4(v, v, v, v);
}
}  // namespace

extern "C" int fv_flush_l2(int device, size_t bytes) {
  // One scratch buffer per device, grown on demand and kept until exit.
  static void* scratch[64] = {nullptr};
  static size_t scratch_bytes[64] = {0};
  FV_REQUIRE(device >= 0 && device < 64, FV_ERR_INVALID, "fv_flush_l2: device %d out of range", device);
  fv::DeviceGuard g(device);
  FV_REQUIRE(g.ok, FV_ERR_CUDA, "fv_flush_l2: cannot select device %d", device);
  bytes = (bytes + 15) & ~(size_t)15;
  if (bytes == 0) return FV_OK;
  if (scratch_bytes[device] < bytes) {
    if (scratch[device]) FV_CUDA(cudaFree(scratch[device]));
    scratch[device] = nullptr;
    scratch_bytes[device] = 0;
    FV_CUDA(cudaMalloc(&scratch[device], bytes));
    scratch_bytes[device] = bytes;
  }
  static uint32_t tick = 0;
  k_flush<<<1184, 256>>>((uint4*)scratch[device], bytes / 16, ++tick);
  FV_CUDA(cudaGetLastError());
  FV_CUDA(cudaDeviceSynchronize());
  return FV_OK;
}

// ---------------------------------------------------------------------------
// Read-bandwidth probe: what this GPU delivers for the two access patterns of the train step, so that
// a kernel's rate can be set beside a figure measured in the same run.
//   pattern 0  streaming: every thread reads 128-bit words with a grid stride, four loads in flight
//   pattern 1  row gather: a warp reads whole rows of `row_bytes` (a multiple of 16) at pseudo-random
//              places of the buffer, four rows in flight -- the shape of the forward pass
// The buffer of `footprint` bytes is read `reps` times after one untimed pass; a footprint below the
// L2 size measures the L2, a much larger one the HBM.
// ---------------------------------------------------------------------------
namespace {
__global__ void __launch_bounds__(256) k_probe_stream(const uint4* __restrict__ p, size_t n, int reps, unsigned* sink) {
  const size_t tid = (size_t)blockIdx.x * blockDim.x + threadIdx.x, nt = (size_t)gridDim.x * blockDim.x;
  unsigned acc = 0;
  for (int r = 0; r < reps; ++r) {
    size_t i = tid;
    for (; i + 3 * nt < n; i += 4 * nt) {
      const uint4 a = __ldcg(p + i), b = __ldcg(p + i + nt), c = __ldcg(p + i + 2 * nt), d = __ldcg(p + i + 3 * nt);
      acc ^= a.x ^ b.y ^ c.z ^ d.w;
    }
    for (; i < n; i += nt) acc ^= __ldcg(p + i).x;
  }
  if (acc == 0x12345678u) *sink = acc;  // keeps the loads alive
}
__global__ void __launch_bounds__(256) k_probe_gather(const uint4* __restrict__ p, unsigned nrows, int row_q, int rows_per_warp,
                                                      unsigned seed, unsigned* sink) {
  const int lane = threadIdx.x & 31;
  const size_t warp = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  unsigned s = seed + (unsigned)warp * 2654435761u, acc = 0;
  for (int k = 0; k < rows_per_warp; k += 4) {
    const uint4* r[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      s = s * 1664525u + 1013904223u;
      r[u] = p + (size_t)((s >> 8) % nrows) * row_q;
    }
    for (int q0 = 0; q0 < row_q; q0 += 128) {
      uint4 v[4][4];
#pragma unroll
      for (int u = 0; u < 4; ++u)
#pragma unroll
        for (int t = 0; t < 4; ++t) {
          const int q = q0 + lane + 32 * t;
          v[u][t] = q < row_q ? __ldcg(r[u] + q) : make_uint4(0u, 0u, 0u, 0u);
        }
#pragma unroll
      for (int u = 0; u < 4; ++u)
#pragma unroll
        for (int t = 0; t < 4; ++t) acc ^= v[u][t].x ^ v[u][t].w;
    }
  }
  if (acc == 0x12345678u) *sink = acc;
}
}  // namespace

extern "C" int fv_probe_read_bandwidth(int device, int pattern, size_t footprint, uint32_t row_bytes, uint32_t reps,
                                       double* gbytes_per_s) {
  FV_REQUIRE(gbytes_per_s != nullptr, FV_ERR_INVALID, "fv_probe_read_bandwidth: output pointer is NULL");
  FV_REQUIRE(pattern == 0 || pattern == 1, FV_ERR_INVALID, "pattern must be 0 (streaming) or 1 (row gather)");
  FV_REQUIRE(footprint >= (1u << 20) && footprint <= ((size_t)8 << 30), FV_ERR_INVALID, "footprint must be between 1 MiB and 8 GiB");
  FV_REQUIRE(reps >= 1 && reps <= 100000, FV_ERR_INVALID, "reps out of range");
  if (pattern == 1) FV_REQUIRE(row_bytes >= 16 && row_bytes % 16 == 0 && row_bytes <= footprint, FV_ERR_INVALID, "row_bytes must be a multiple of 16");
  fv::DeviceGuard g(device);
  FV_REQUIRE(g.ok, FV_ERR_CUDA, "cannot select device %d", device);
  cudaDeviceProp prop;
  FV_CUDA(cudaGetDeviceProperties(&prop, device));
  void* buf = nullptr;
  unsigned* sink = nullptr;
  cudaEvent_t e0 = nullptr, e1 = nullptr;
  FV_CUDA(cudaMalloc(&buf, footprint));
  cudaError_t e = cudaMalloc((void**)&sink, sizeof(unsigned));
  if (e == cudaSuccess) e = cudaMemset(buf, 1, footprint);
  if (e == cudaSuccess) e = cudaEventCreate(&e0);
  if (e == cudaSuccess) e = cudaEventCreate(&e1);
  double bytes = 0.0;
  float ms = 0.f;
  if (e == cudaSuccess) {
    const int grid = prop.multiProcessorCount * 8;
    if (pattern == 0) {
      const size_t n = footprint / 16;
      k_probe_stream<<<grid, 256>>>(static_cast<const uint4*>(buf), n, 1, sink);
      cudaEventRecord(e0);
      k_probe_stream<<<grid, 256>>>(static_cast<const uint4*>(buf), n, (int)reps, sink);
      cudaEventRecord(e1);
      bytes = (double)n * 16.0 * reps;
    } else {
      const unsigned nrows = (unsigned)(footprint / row_bytes);
      const int row_q = (int)(row_bytes / 16);
      // reps full passes' worth of rows, spread over the warps
      const size_t warps = (size_t)grid * 8;
      size_t per_warp = ((size_t)nrows * reps + warps - 1) / warps;
      per_warp = (per_warp + 3) & ~(size_t)3;
      k_probe_gather<<<grid, 256>>>(static_cast<const uint4*>(buf), nrows, row_q, 64, 1u, sink);
      cudaEventRecord(e0);
      k_probe_gather<<<grid, 256>>>(static_cast<const uint4*>(buf), nrows, row_q, (int)per_warp, 7u, sink);
      cudaEventRecord(e1);
      bytes = (double)warps * (double)per_warp * (double)row_bytes;
    }
    e = cudaGetLastError();
    if (e == cudaSuccess) e = cudaEventSynchronize(e1);
    if (e == cudaSuccess) e = cudaEventElapsedTime(&ms, e0, e1);
  }
  if (e0) cudaEventDestroy(e0);
  if (e1) cudaEventDestroy(e1);
  cudaFree(sink);
  cudaFree(buf);
  FV_CUDA(e);
  *gbytes_per_s = bytes / ((double)ms * 1e-3) / 1e9;
  return FV_OK;
}
