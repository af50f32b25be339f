// FlyVec hasher for sm_100a.
//
// The synapse matrix is held transposed, wt[N][Kp] (row = one input id, Kp = K
// padded to a multiple of 4), optionally row-normalised exactly as the
// reference does it (flyvec/core.py:22-36).  A code is computed by one warp:
// activations of the K units -> the hash_length-th and the next largest value
// by a bitwise search on order-preserving integer keys -> threshold at their
// float midpoint with a strict '>' (flyvec/core.py:155-158) -> bits.
#include <cmath>
#include <cstring>
#include <vector>

#include <algorithm>

#include "fv_common.h"

namespace {

constexpr unsigned FULL = 0xffffffffu;

struct HDev {
  int K, Kp, Kq, N, V;
  const float* wt;
  const float* f;  // 1/count per vocabulary id, may be null
  uint32_t* error;
  float wabsmax;   // max |wt| (bounds the rounding error of the float window sums)
  float fmax;      // max |f|
};

// ---- normalisation ---------------------------------------------------------
// numpy sums a contiguous float32 row pairwise: blocks of at most 128 elements
// are summed with eight interleaved accumulators combined as
// ((r0+r1)+(r2+r3))+((r4+r5)+(r6+r7)) plus a sequential tail; longer ranges are
// split at n/2 rounded down to a multiple of 8.  np.sum(syn**2, axis=1) in
// flyvec/core.py:35 therefore has a fixed association order, reproduced here so
// that the normalised weights -- and every code derived from them -- are
// bit-identical to the reference's.
__device__ float leaf_sumsq(const float* __restrict__ a, long long n) {
  if (n < 8) {
    float r = 0.f;
    for (long long i = 0; i < n; ++i) r = __fadd_rn(r, __fmul_rn(a[i], a[i]));
    return r;
  }
  float r[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) r[j] = __fmul_rn(a[j], a[j]);
  long long i = 8;
  const long long m = n - (n % 8);
  for (; i < m; i += 8) {
#pragma unroll
    for (int j = 0; j < 8; ++j) r[j] = __fadd_rn(r[j], __fmul_rn(a[i + j], a[i + j]));
  }
  float res = __fadd_rn(__fadd_rn(__fadd_rn(r[0], r[1]), __fadd_rn(r[2], r[3])),
                        __fadd_rn(__fadd_rn(r[4], r[5]), __fadd_rn(r[6], r[7])));
  for (; i < n; ++i) res = __fadd_rn(res, __fmul_rn(a[i], a[i]));
  return res;
}

// Post-order walk of the split tree with an explicit stack (depth <= log2(n/64)).
__device__ float pairwise_sumsq(const float* __restrict__ a, long long n) {
  struct Frame {
    long long off, n;
    float lo;
    int stage;
  };
  Frame st[40];
  int sp = 0;
  st[0] = Frame{0, n, 0.f, 0};
  float ret = 0.f;
  while (sp >= 0) {
    Frame& fr = st[sp];
    if (fr.stage == 0) {
      if (fr.n <= 128) {
        ret = leaf_sumsq(a + fr.off, fr.n);
        --sp;
        continue;
      }
      long long n2 = fr.n / 2;
      n2 -= n2 % 8;
      fr.stage = 1;
      st[sp + 1] = Frame{fr.off, n2, 0.f, 0};
      ++sp;
    } else if (fr.stage == 1) {
      long long n2 = fr.n / 2;
      n2 -= n2 % 8;
      fr.lo = ret;
      fr.stage = 2;
      st[sp + 1] = Frame{fr.off + n2, fr.n - n2, 0.f, 0};
      ++sp;
    } else {
      ret = __fadd_rn(fr.lo, ret);
      --sp;
    }
  }
  return ret;
}

// One thread per unit: norm[mu] = sqrt(sum_i w[mu][i]^2) + prec, all in float.
__global__ void k_row_norms(const float* __restrict__ w_kn, int K, long long N, float prec, float* __restrict__ norm) {
  const int mu = blockIdx.x * blockDim.x + threadIdx.x;
  if (mu >= K) return;
  const float ss = pairwise_sumsq(w_kn + (size_t)mu * N, N);
  norm[mu] = __fadd_rn(__fsqrt_rn(ss), prec);
}

// max |x| over n floats as a bit pattern (non-negative floats order like their bits)
__global__ void k_absmax_bits(const float* __restrict__ x, size_t n, uint32_t* __restrict__ out) {
  uint32_t m = 0u;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
    m = max(m, __float_as_uint(x[i]) & 0x7fffffffu);
  m = __reduce_max_sync(FULL, m);
  if ((threadIdx.x & 31) == 0 && m) atomicMax(out, m);
}

// [K][N] -> [N][Kp], dividing by the unit's norm when norm != nullptr.
__global__ void k_load_transposed(const float* __restrict__ w_kn, const float* __restrict__ norm,
                                  float* __restrict__ wt, int K, int Kp, int N) {
  __shared__ float tile[32][33];
  const int i0 = blockIdx.x * 32, m0 = blockIdx.y * 32;
  for (int r = threadIdx.y; r < 32; r += blockDim.y) {
    const int mu = m0 + r, i = i0 + threadIdx.x;
    float v = 0.f;
    if (mu < K && i < N) {
      v = w_kn[(size_t)mu * N + i];
      if (norm) v = __fdiv_rn(v, norm[mu]);
    }
    tile[r][threadIdx.x] = v;
  }
  __syncthreads();
  for (int r = threadIdx.y; r < 32; r += blockDim.y) {
    const int i = i0 + r, mu = m0 + threadIdx.x;
    if (i < N && mu < Kp) wt[(size_t)i * Kp + mu] = tile[threadIdx.x][r];
  }
}
__global__ void k_store_untransposed(const float* __restrict__ wt, float* __restrict__ w_kn, int K, int Kp, int N) {
  __shared__ float tile[32][33];
  const int i0 = blockIdx.x * 32, m0 = blockIdx.y * 32;
  for (int r = threadIdx.y; r < 32; r += blockDim.y) {
    const int i = i0 + r, mu = m0 + threadIdx.x;
    tile[r][threadIdx.x] = (i < N && mu < K) ? wt[(size_t)i * Kp + mu] : 0.f;
  }
  __syncthreads();
  for (int r = threadIdx.y; r < 32; r += blockDim.y) {
    const int mu = m0 + r, i = i0 + threadIdx.x;
    if (mu < K && i < N) w_kn[(size_t)mu * N + i] = tile[threadIdx.x][r];
  }
}

// ---- selection -------------------------------------------------------------
// Monotone map float -> uint32 (larger float = larger key); 0 is below every
// non-NaN value and marks the padding columns.
__device__ __forceinline__ uint32_t f2key(float x) {
  const uint32_t u = __float_as_uint(x);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ float key2f(uint32_t k) {
  return __uint_as_float((k & 0x80000000u) ? (k & 0x7fffffffu) : ~k);
}

// MODE 0: token ids (activation = row V+id); MODE 1: windows, weighted by f;
// MODE 2: windows, raw.
template <int NT, int MODE>
__global__ void __launch_bounds__(256, (NT <= 4) ? 3 : 1) k_hash(HDev h, const int32_t* __restrict__ in, unsigned long long n, int W,
                                              int hash_len, uint32_t flags, uint8_t* __restrict__ out) {
  const int lane = threadIdx.x & 31;
  const unsigned long long warp = ((unsigned long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const unsigned long long nwarps = ((unsigned long long)gridDim.x * blockDim.x) >> 5;
  const int Kq = h.Kq;
  const bool bytes_out = (flags & FV_HASH_BYTES) != 0;
  const size_t out_stride = bytes_out ? (size_t)h.K : (size_t)((h.K + 7) / 8);
  // Bound on |float window sum - reference window sum| for a window whose terms are bounded by
  // t_c = f_c * max|wt|: sequential float summation is off by at most (W-1) * 2^-24 * sum t_c, product
  // rounding (one fused rounding here, a rounded product there) and the final float store add at most
  // 3 * 2^-24 * sum t_c; times four for safety.  theta = theta_unit * sum f_c is formed per window.
  const float theta_unit = 4.0f * (float)(W + 2) * 5.9604645e-8f * h.wabsmax;
  const bool exact_only = (flags & FV_HASH_EXACT) != 0;

  for (unsigned long long item = warp; item < n; item += nwarps) {
    float a[NT][4];
    bool zero_code = false;
    if (MODE == 0) {
      const int id = in[item];
      if (id < 0 || id >= h.V) {
        if (lane == 0) atomicOr(h.error, FV_DEVERR_TOKEN_RANGE);
        zero_code = true;
      } else if (id == 0 && !(flags & FV_HASH_NO_UNK)) {
        zero_code = true;  // the unknown token hashes to all zeros (flyvec/core.py:120-125, 151)
      }
      const float4* __restrict__ row =
          reinterpret_cast<const float4*>(h.wt + (size_t)(h.V + (zero_code ? 0 : id)) * h.Kp);
#pragma unroll
      for (int t = 0; t < NT; ++t) {
        const int q = lane + 32 * t;
        const float4 v = (q < Kq) ? __ldg(row + q) : make_float4(0.f, 0.f, 0.f, 0.f);
        a[t][0] = v.x; a[t][1] = v.y; a[t][2] = v.z; a[t][3] = v.w;
      }
    }
    // Window sums.  The reference adds the (float) terms in double and stores a float
    // (flyvec/src/cuda_funcs.cu:289-305; 248-263 for the raw form).  Converting every term to double
    // is what bounds this kernel, so the sums are first formed in float: they are off by at most theta
    // from the reference's, and when the hash_len-th and the next largest of them lie more than
    // 4 * theta apart, the units above the threshold are the same whichever sums are used -- the code
    // is certified.  Otherwise (ties, close calls: well under 1 % of the windows) the warp redoes the
    // window with the reference's arithmetic.
    const int my = (MODE != 0 && lane < W) ? in[item * (unsigned long long)W + lane] : -1;
    if (MODE != 0 && my >= h.N) atomicOr(h.error, FV_DEVERR_TOKEN_RANGE);
    bool done = false;
    uint32_t kh = 0u;
    float thr = 0.f, theta = 0.f;
    for (int pass = (MODE == 0 || exact_only) ? 1 : 0; pass < 2 && !done; ++pass) {
      if (MODE != 0 && pass == 0) {
        float acc[NT][4];
#pragma unroll
        for (int t = 0; t < NT; ++t) acc[t][0] = acc[t][1] = acc[t][2] = acc[t][3] = 0.f;
        for (int c0 = 0; c0 < W; c0 += 4) {  // four rows' loads in flight together
          const float4* __restrict__ row[4];
          float sc[4];
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            const int id = __shfl_sync(FULL, my, (c0 + u) & 31);
            const bool ok = c0 + u < W && id >= 0 && id < h.N;
            row[u] = reinterpret_cast<const float4*>(h.wt + (size_t)(ok ? id : 0) * h.Kp);
            sc[u] = !ok ? 0.f : (MODE == 1) ? __ldg(h.f + (id % h.V)) : 1.f;  // an absent position adds 0 * (row 0)
            theta += theta_unit * fabsf(sc[u]);
          }
          float4 v[4][NT];
#pragma unroll
          for (int u = 0; u < 4; ++u)
#pragma unroll
            for (int t = 0; t < NT; ++t) v[u][t] = __ldg(row[u] + min(lane + 32 * t, Kq - 1));
#pragma unroll
          for (int u = 0; u < 4; ++u)
#pragma unroll
            for (int t = 0; t < NT; ++t) {
              acc[t][0] = fmaf(v[u][t].x, sc[u], acc[t][0]);
              acc[t][1] = fmaf(v[u][t].y, sc[u], acc[t][1]);
              acc[t][2] = fmaf(v[u][t].z, sc[u], acc[t][2]);
              acc[t][3] = fmaf(v[u][t].w, sc[u], acc[t][3]);
            }
        }
#pragma unroll
        for (int t = 0; t < NT; ++t)
#pragma unroll
          for (int k = 0; k < 4; ++k) a[t][k] = acc[t][k];
      } else if (MODE != 0) {
        double acc[NT][4];
#pragma unroll
        for (int t = 0; t < NT; ++t) acc[t][0] = acc[t][1] = acc[t][2] = acc[t][3] = 0.0;
        for (int c = 0; c < W; ++c) {
          const int id = __shfl_sync(FULL, my, c);
          if (id < 0 || id >= h.N) continue;
          const float sc = (MODE == 1) ? __ldg(h.f + (id % h.V)) : 1.f;
          const float4* __restrict__ row = reinterpret_cast<const float4*>(h.wt + (size_t)id * h.Kp);
#pragma unroll
          for (int t = 0; t < NT; ++t) {
            const int q = lane + 32 * t;
            if (q < Kq) {
              const float4 v = __ldg(row + q);
              if (MODE == 1) {
                acc[t][0] += (double)__fmul_rn(v.x, sc);
                acc[t][1] += (double)__fmul_rn(v.y, sc);
                acc[t][2] += (double)__fmul_rn(v.z, sc);
                acc[t][3] += (double)__fmul_rn(v.w, sc);
              } else {
                acc[t][0] += (double)v.x;
                acc[t][1] += (double)v.y;
                acc[t][2] += (double)v.z;
                acc[t][3] += (double)v.w;
              }
            }
          }
        }
#pragma unroll
        for (int t = 0; t < NT; ++t)
#pragma unroll
          for (int k = 0; k < 4; ++k) a[t][k] = (float)acc[t][k];
      }

      uint32_t key[NT][4];
      uint32_t kand = 0xffffffffu, kor = 0u;
#pragma unroll
      for (int t = 0; t < NT; ++t)
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const bool real = 4 * (lane + 32 * t) + k < h.K;
          key[t][k] = real ? f2key(a[t][k]) : 0u;
          if (real) {
            kand &= key[t][k];
            kor |= key[t][k];
          }
        }
      // hash_len-th largest key: the largest v with #{key >= v} >= hash_len, found bit by bit; the
      // leading bits all keys share (sign and most of the exponent, as a rule) need no search
      kand = __reduce_and_sync(FULL, kand);
      kor = __reduce_or_sync(FULL, kor);
      const int shared_bits = __clz(kand ^ kor);  // 32 when all keys are equal
      kh = shared_bits >= 32 ? kand : (kand & ~(0xffffffffu >> shared_bits));
      bool split = false;  // a candidate with exactly hash_len keys at or above it separates the two order statistics
      for (int bit = 31 - shared_bits; bit >= 0 && !split; --bit) {
        const uint32_t cand = kh | (1u << bit);
        int c = 0;
#pragma unroll
        for (int t = 0; t < NT; ++t)
#pragma unroll
          for (int k = 0; k < 4; ++k) c += (key[t][k] >= cand);
        c = __reduce_add_sync(FULL, c);
        if (c >= hash_len) kh = cand;
        split = (c == hash_len);
      }
      uint32_t kn;
      if (split) {
        // kh is a lower bound with exactly hash_len keys at or above it: the hash_len-th largest is the
        // smallest of those, the next one the largest below (the remaining bits need no search)
        uint32_t above = 0xffffffffu, below = 0u;
#pragma unroll
        for (int t = 0; t < NT; ++t)
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            if (key[t][k] >= kh) above = min(above, key[t][k]);
            else below = max(below, key[t][k]);
          }
        kh = __reduce_min_sync(FULL, above);
        kn = __reduce_max_sync(FULL, below);
      } else {
        // ties at the hash_len-th value: kh is that value; the next one in sorted order is kh again if it
        // occurs beyond rank hash_len, else the largest key below it
        int cge = 0;
        uint32_t below = 0u;
#pragma unroll
        for (int t = 0; t < NT; ++t)
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            cge += (key[t][k] >= kh);
            if (key[t][k] < kh) below = max(below, key[t][k]);
          }
        cge = __reduce_add_sync(FULL, cge);
        below = __reduce_max_sync(FULL, below);
        kn = (cge > hash_len) ? kh : below;
      }
      thr = __fmul_rn(__fadd_rn(key2f(kh), key2f(kn)), 0.5f);
      // pass 0 only stands when the two order statistics are clearly apart (NaN compares false)
      done = (pass == 1) || (key2f(kh) - key2f(kn) > 4.0f * theta);
    }

    uint8_t* __restrict__ dst = out + (size_t)item * out_stride;
#pragma unroll
    for (int t = 0; t < NT; ++t) {
      const int q = lane + 32 * t;
      uint32_t nib = 0u;
#pragma unroll
      for (int k = 0; k < 4; ++k)
        if (!zero_code && 4 * q + k < h.K && a[t][k] > thr) nib |= 1u << k;
      if (bytes_out) {
#pragma unroll
        for (int k = 0; k < 4; ++k)
          if (4 * q + k < h.K) dst[4 * q + k] = (uint8_t)((nib >> k) & 1u);
      } else {
        const uint32_t hi = __shfl_down_sync(FULL, nib, 1);
        if (!(lane & 1) && 4 * q < h.K) dst[q >> 1] = (uint8_t)(nib | (hi << 4));
      }
    }
  }
}

// A vocabulary has only V distinct token codes.  For a batch much larger than V the codes of all
// ids are computed once into a table (k_hash over 0..V-1) and the batch becomes a gather of
// `stride` bytes per token; the table (1 MB at V = 20000, bit-packed) stays in L2.
__global__ void k_iota32(int32_t* p, int n) {
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) p[i] = i;
}
template <typename T>
__global__ void __launch_bounds__(256) k_gather_codes(const uint8_t* __restrict__ table, const int32_t* __restrict__ ids,
                                                      unsigned long long n, int V, int stride, uint8_t* __restrict__ out,
                                                      uint32_t* error) {
  const int lane = threadIdx.x & 31;
  const unsigned long long warp = ((unsigned long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const unsigned long long nwarps = ((unsigned long long)gridDim.x * blockDim.x) >> 5;
  const int per = stride / (int)sizeof(T);
  for (unsigned long long item = warp; item < n; item += nwarps) {
    int id = ids[item];
    if (id < 0 || id >= V) {
      if (lane == 0) atomicOr(error, FV_DEVERR_TOKEN_RANGE);
      id = 0;
    }
    const T* __restrict__ src = reinterpret_cast<const T*>(table + (size_t)id * stride);
    T* __restrict__ dst = reinterpret_cast<T*>(out + (size_t)item * stride);
    for (int k = lane; k < per; k += 32) dst[k] = src[k];
  }
}

}  // namespace

struct fv_hasher {
  int device = 0;
  int num_sms = 0;
  int NT = 1;
  HDev h;
  float* d_wt = nullptr;
  float* d_f = nullptr;
  uint32_t* d_err = nullptr;
  cudaStream_t stream = nullptr;
  cudaEvent_t ev0 = nullptr, ev1 = nullptr;
  // codes of the whole vocabulary for one (hash length, format), kept between calls
  uint8_t* d_table = nullptr;
  int32_t* d_iota = nullptr;
  uint32_t table_hl = 0, table_flags = 0xffffffffu;
  // host-buffer calls: two pipeline slots, each a stream with device and pinned staging buffers (made on first use)
  cudaStream_t pipe_stream[2] = {nullptr, nullptr};
  cudaEvent_t pipe_done[2] = {nullptr, nullptr};
  int32_t* pipe_d_in[2] = {nullptr, nullptr};
  uint8_t* pipe_d_out[2] = {nullptr, nullptr};
  int32_t* pipe_h_in[2] = {nullptr, nullptr};
  uint8_t* pipe_h_out[2] = {nullptr, nullptr};
  size_t pipe_bytes = 0;
};

namespace {

#define FV_TRY(expr)                    \
  do {                                  \
    int fv_rc_ = (expr);                \
    if (fv_rc_ != FV_OK) return fv_rc_; \
  } while (0)

template <int NT>
void launch_hash(fv_hasher* hs, cudaStream_t stream, int mode, int grid, const int32_t* in, unsigned long long n, int W, int hl,
                 uint32_t flags, uint8_t* out) {
  if (mode == 0)
    k_hash<NT, 0><<<grid, 256, 0, stream>>>(hs->h, in, n, W, hl, flags, out);
  else if (mode == 1)
    k_hash<NT, 1><<<grid, 256, 0, stream>>>(hs->h, in, n, W, hl, flags, out);
  else
    k_hash<NT, 2><<<grid, 256, 0, stream>>>(hs->h, in, n, W, hl, flags, out);
}

// The hashing kernel for n items on `stream`; no synchronisation, the device error word only collects.
void enqueue_hash(fv_hasher* hs, cudaStream_t stream, int mode, const int32_t* d_in, unsigned long long n, int W, uint32_t hash_len,
                  uint32_t flags, uint8_t* d_out) {
  const unsigned long long blocks = (n + 7) / 8;
  const unsigned long long cap = (unsigned long long)hs->num_sms * 8;
  const int grid = (int)(blocks < cap ? blocks : cap);
  switch (hs->NT) {
    case 1: launch_hash<1>(hs, stream, mode, grid, d_in, n, W, (int)hash_len, flags, d_out); break;
    case 2: launch_hash<2>(hs, stream, mode, grid, d_in, n, W, (int)hash_len, flags, d_out); break;
    case 3: launch_hash<3>(hs, stream, mode, grid, d_in, n, W, (int)hash_len, flags, d_out); break;
    case 4: launch_hash<4>(hs, stream, mode, grid, d_in, n, W, (int)hash_len, flags, d_out); break;
    case 5: launch_hash<5>(hs, stream, mode, grid, d_in, n, W, (int)hash_len, flags, d_out); break;
    case 6: launch_hash<6>(hs, stream, mode, grid, d_in, n, W, (int)hash_len, flags, d_out); break;
    case 7: launch_hash<7>(hs, stream, mode, grid, d_in, n, W, (int)hash_len, flags, d_out); break;
    default: launch_hash<8>(hs, stream, mode, grid, d_in, n, W, (int)hash_len, flags, d_out); break;
  }
}

// Codes of n token ids gathered from the vocabulary table on `stream` (the table must be current).
void enqueue_gather(fv_hasher* hs, cudaStream_t stream, const int32_t* d_in, unsigned long long n, int stride, uint8_t* d_out) {
  const HDev& h = hs->h;
  const unsigned long long blocks = (n + 7) / 8;
  const unsigned long long cap = (unsigned long long)hs->num_sms * 16;
  const int grid = (int)(blocks < cap ? blocks : cap);
  if (stride % 16 == 0)
    k_gather_codes<uint4><<<grid, 256, 0, stream>>>(hs->d_table, d_in, n, h.V, stride, d_out, hs->d_err);
  else if (stride % 4 == 0)
    k_gather_codes<uint32_t><<<grid, 256, 0, stream>>>(hs->d_table, d_in, n, h.V, stride, d_out, hs->d_err);
  else if (stride % 2 == 0)
    k_gather_codes<uint16_t><<<grid, 256, 0, stream>>>(hs->d_table, d_in, n, h.V, stride, d_out, hs->d_err);
  else
    k_gather_codes<uint8_t><<<grid, 256, 0, stream>>>(hs->d_table, d_in, n, h.V, stride, d_out, hs->d_err);
}

int run_hash(fv_hasher* hs, int mode, const int32_t* d_in, unsigned long long n, int W, uint32_t hash_len,
             uint32_t flags, uint8_t* d_out, double* seconds, bool may_allocate = true);

// Token hashing through the vocabulary table.  Builds (or reuses) the table, then gathers.
int run_hash_table(fv_hasher* hs, const int32_t* d_in, unsigned long long n, uint32_t hash_len, uint32_t flags,
                   uint8_t* d_out, double* seconds) {
  const HDev& h = hs->h;
  const int stride = (flags & FV_HASH_BYTES) ? h.K : (h.K + 7) / 8;
  const uint32_t key_flags = flags & (FV_HASH_BYTES | FV_HASH_NO_UNK);
  if (!hs->d_table || hs->table_hl != hash_len || hs->table_flags != key_flags) {
    if (!hs->d_iota) {
      FV_CUDA(cudaMalloc((void**)&hs->d_iota, (size_t)h.V * sizeof(int32_t)));
      k_iota32<<<64, 256, 0, hs->stream>>>(hs->d_iota, h.V);
      FV_CUDA(cudaGetLastError());
    }
    if (hs->d_table && (hs->table_flags & FV_HASH_BYTES) != (key_flags & FV_HASH_BYTES)) {
      FV_CUDA(cudaFree(hs->d_table));
      hs->d_table = nullptr;
    }
    if (!hs->d_table) FV_CUDA(cudaMalloc((void**)&hs->d_table, (size_t)h.V * stride));
    hs->table_flags = 0xffffffffu;
    const int rc = run_hash(hs, 0, hs->d_iota, (unsigned long long)h.V, 0, hash_len, key_flags, hs->d_table, nullptr, false);
    if (rc != FV_OK) return rc;
    hs->table_hl = hash_len;
    hs->table_flags = key_flags;
  }
  if (!d_in) return FV_OK;  // the caller only wanted the table
  FV_CUDA(cudaMemsetAsync(hs->d_err, 0, sizeof(uint32_t), hs->stream));
  FV_CUDA(cudaEventRecord(hs->ev0, hs->stream));
  enqueue_gather(hs, hs->stream, d_in, n, stride, d_out);
  FV_CUDA(cudaGetLastError());
  FV_CUDA(cudaEventRecord(hs->ev1, hs->stream));
  uint32_t err = 0;
  FV_CUDA(cudaMemcpyAsync(&err, hs->d_err, sizeof(err), cudaMemcpyDeviceToHost, hs->stream));
  FV_CUDA(cudaStreamSynchronize(hs->stream));
  if (seconds) {
    float ms = 0.f;
    FV_CUDA(cudaEventElapsedTime(&ms, hs->ev0, hs->ev1));
    *seconds = ms * 1e-3;
  }
  if (err & FV_DEVERR_TOKEN_RANGE) return fv::fail(FV_ERR_DATA, "an input id was out of range (device check)");
  return FV_OK;
}

int run_hash(fv_hasher* hs, int mode, const int32_t* d_in, unsigned long long n, int W, uint32_t hash_len,
             uint32_t flags, uint8_t* d_out, double* seconds, bool may_allocate) {
  FV_REQUIRE(hash_len >= 1 && (int)hash_len < hs->h.K, FV_ERR_INVALID,
             "hash_length must be in [1, K-1] (K = %d), got %u", hs->h.K, hash_len);
  if (seconds) *seconds = 0.0;
  if (n == 0) return FV_OK;
  // many more tokens than vocabulary entries: hash the vocabulary once, then gather
  if (mode == 0 && may_allocate && n >= 4ull * (unsigned long long)hs->h.V)
    return run_hash_table(hs, d_in, n, hash_len, flags, d_out, seconds);
  FV_CUDA(cudaMemsetAsync(hs->d_err, 0, sizeof(uint32_t), hs->stream));
  FV_CUDA(cudaEventRecord(hs->ev0, hs->stream));
  enqueue_hash(hs, hs->stream, mode, d_in, n, W, hash_len, flags, d_out);
  FV_CUDA(cudaGetLastError());
  FV_CUDA(cudaEventRecord(hs->ev1, hs->stream));
  uint32_t err = 0;
  FV_CUDA(cudaMemcpyAsync(&err, hs->d_err, sizeof(err), cudaMemcpyDeviceToHost, hs->stream));
  FV_CUDA(cudaStreamSynchronize(hs->stream));
  if (seconds) {
    float ms = 0.f;
    FV_CUDA(cudaEventElapsedTime(&ms, hs->ev0, hs->ev1));
    *seconds = ms * 1e-3;
  }
  if (err & FV_DEVERR_TOKEN_RANGE) return fv::fail(FV_ERR_DATA, "an input id was out of range (device check)");
  return FV_OK;
}

void free_hasher(fv_hasher* hs) {
  cudaSetDevice(hs->device);
  if (hs->d_wt) cudaFree(hs->d_wt);
  if (hs->d_f) cudaFree(hs->d_f);
  if (hs->d_err) cudaFree(hs->d_err);
  if (hs->d_table) cudaFree(hs->d_table);
  if (hs->d_iota) cudaFree(hs->d_iota);
  if (hs->ev0) cudaEventDestroy(hs->ev0);
  if (hs->ev1) cudaEventDestroy(hs->ev1);
  if (hs->stream) cudaStreamDestroy(hs->stream);
  for (int b = 0; b < 2; ++b) {
    if (hs->pipe_d_in[b]) cudaFree(hs->pipe_d_in[b]);
    if (hs->pipe_d_out[b]) cudaFree(hs->pipe_d_out[b]);
    if (hs->pipe_h_in[b]) cudaFreeHost(hs->pipe_h_in[b]);
    if (hs->pipe_h_out[b]) cudaFreeHost(hs->pipe_h_out[b]);
    if (hs->pipe_done[b]) cudaEventDestroy(hs->pipe_done[b]);
    if (hs->pipe_stream[b]) cudaStreamDestroy(hs->pipe_stream[b]);
  }
  delete hs;
}

int create_hasher(fv_hasher* hs, const float* w_kn, int K, int N, int normalize, float prec, int device) {
  hs->device = device;
  FV_CUDA(cudaSetDevice(device));
  cudaDeviceProp prop;
  FV_CUDA(cudaGetDeviceProperties(&prop, device));
  hs->num_sms = prop.multiProcessorCount;
  FV_CUDA(cudaStreamCreateWithFlags(&hs->stream, cudaStreamNonBlocking));
  FV_CUDA(cudaEventCreate(&hs->ev0));
  FV_CUDA(cudaEventCreate(&hs->ev1));
  HDev& h = hs->h;
  h.K = K;
  h.Kp = (K + 3) & ~3;
  h.Kq = h.Kp / 4;
  h.N = N;
  h.V = N / 2;
  h.f = nullptr;
  hs->NT = (h.Kq + 31) / 32;
  FV_CUDA(cudaMalloc((void**)&hs->d_wt, (size_t)N * h.Kp * sizeof(float)));
  FV_CUDA(cudaMalloc((void**)&hs->d_err, sizeof(uint32_t)));
  h.wt = hs->d_wt;
  h.error = hs->d_err;
  float* tmp = nullptr;
  float* norm = nullptr;
  FV_CUDA(cudaMalloc((void**)&tmp, (size_t)K * N * sizeof(float)));
  cudaError_t e = cudaMemcpyAsync(tmp, w_kn, (size_t)K * N * sizeof(float), cudaMemcpyHostToDevice, hs->stream);
  if (e == cudaSuccess && normalize) {
    e = cudaMalloc((void**)&norm, (size_t)K * sizeof(float));
    if (e == cudaSuccess) {
      k_row_norms<<<(K + 31) / 32, 32, 0, hs->stream>>>(tmp, K, (long long)N, prec, norm);
      e = cudaGetLastError();
    }
  }
  if (e == cudaSuccess) {
    dim3 grid((N + 31) / 32, (h.Kp + 31) / 32), block(32, 8);
    k_load_transposed<<<grid, block, 0, hs->stream>>>(tmp, norm, hs->d_wt, K, h.Kp, N);
    e = cudaGetLastError();
  }
  uint32_t wmax_bits = 0u;
  if (e == cudaSuccess) e = cudaMemsetAsync(hs->d_err, 0, sizeof(uint32_t), hs->stream);
  if (e == cudaSuccess) {
    k_absmax_bits<<<hs->num_sms * 4, 256, 0, hs->stream>>>(hs->d_wt, (size_t)N * h.Kp, hs->d_err);  // d_err as scratch
    e = cudaGetLastError();
  }
  if (e == cudaSuccess) e = cudaMemcpyAsync(&wmax_bits, hs->d_err, sizeof(uint32_t), cudaMemcpyDeviceToHost, hs->stream);
  if (e == cudaSuccess) e = cudaMemsetAsync(hs->d_err, 0, sizeof(uint32_t), hs->stream);
  if (e == cudaSuccess) e = cudaStreamSynchronize(hs->stream);
  cudaFree(tmp);
  if (norm) cudaFree(norm);
  FV_CUDA(e);
  memcpy(&h.wabsmax, &wmax_bits, sizeof(float));  // NaN or infinity here sends every window to the exact pass
  h.fmax = 1.0f;
  return FV_OK;
}

}  // namespace

extern "C" {

int fv_hasher_create(const float* w_kn, uint32_t hid, uint32_t n_cols, int normalize, float prec, int device,
                     fv_hasher** out) {
  FV_REQUIRE(w_kn && out, FV_ERR_INVALID, "fv_hasher_create: NULL argument");
  *out = nullptr;
  FV_REQUIRE(hid >= 2 && hid <= 1024, FV_ERR_INVALID, "hid must be in [2, 1024], got %u", hid);
  FV_REQUIRE(n_cols >= 2 && n_cols % 2 == 0 && n_cols <= (1u << 30), FV_ERR_INVALID,
             "the synapse matrix needs an even number of columns (context half, target half), got %u", n_cols);
  int ndev = 0;
  FV_CUDA(cudaGetDeviceCount(&ndev));
  FV_REQUIRE(device >= 0 && device < ndev, FV_ERR_INVALID, "device %d not present (%d devices)", device, ndev);
  int prev = 0;
  cudaGetDevice(&prev);
  fv_hasher* hs = new fv_hasher();
  const int rc = create_hasher(hs, w_kn, (int)hid, (int)n_cols, normalize, prec, device);
  if (rc != FV_OK) {
    free_hasher(hs);
    cudaSetDevice(prev);
    return rc;
  }
  cudaSetDevice(prev);
  *out = hs;
  return FV_OK;
}

int fv_hasher_destroy(fv_hasher* h) {
  if (!h) return FV_OK;
  int prev = 0;
  cudaGetDevice(&prev);
  cudaSetDevice(h->device);
  cudaDeviceSynchronize();
  free_hasher(h);
  cudaSetDevice(prev);
  return FV_OK;
}

int fv_hasher_get_weights(fv_hasher* hs, float* w_kn) {
  FV_REQUIRE(hs && w_kn, FV_ERR_INVALID, "fv_hasher_get_weights: NULL argument");
  fv::DeviceGuard guard(hs->device);
  const HDev& h = hs->h;
  float* tmp = nullptr;
  FV_CUDA(cudaMalloc((void**)&tmp, (size_t)h.K * h.N * sizeof(float)));
  dim3 grid((h.N + 31) / 32, (h.Kp + 31) / 32), block(32, 8);
  k_store_untransposed<<<grid, block, 0, hs->stream>>>(h.wt, tmp, h.K, h.Kp, h.N);
  cudaError_t e = cudaGetLastError();
  if (e == cudaSuccess)
    e = cudaMemcpyAsync(w_kn, tmp, (size_t)h.K * h.N * sizeof(float), cudaMemcpyDeviceToHost, hs->stream);
  if (e == cudaSuccess) e = cudaStreamSynchronize(hs->stream);
  cudaFree(tmp);
  FV_CUDA(e);
  return FV_OK;
}

int fv_hasher_set_inverse_frequency(fv_hasher* hs, const float* inv_freq, uint32_t vocab) {
  FV_REQUIRE(hs && inv_freq, FV_ERR_INVALID, "fv_hasher_set_inverse_frequency: NULL argument");
  FV_REQUIRE((int)vocab == hs->h.V, FV_ERR_INVALID, "inverse frequency table has %u entries, vocabulary is %d", vocab,
             hs->h.V);
  fv::DeviceGuard guard(hs->device);
  if (!hs->d_f) FV_CUDA(cudaMalloc((void**)&hs->d_f, (size_t)vocab * sizeof(float)));
  FV_CUDA(cudaMemcpy(hs->d_f, inv_freq, (size_t)vocab * sizeof(float), cudaMemcpyHostToDevice));
  hs->h.f = hs->d_f;
  float fmax = 0.f;
  for (uint32_t v = 0; v < vocab; ++v) fmax = std::fmax(fmax, std::fabs(inv_freq[v]));  // NaN-propagating enough: NaN f gives NaN sums
  hs->h.fmax = fmax;
  return FV_OK;
}

int fv_hash_tokens_device(fv_hasher* hs, const int32_t* d_ids, uint64_t n, uint32_t hash_length, uint32_t flags,
                          uint8_t* d_out, double* kernel_seconds) {
  FV_REQUIRE(hs && (n == 0 || (d_ids && d_out)), FV_ERR_INVALID, "fv_hash_tokens_device: NULL argument");
  fv::DeviceGuard guard(hs->device);
  return run_hash(hs, 0, d_ids, n, 0, hash_length, flags, d_out, kernel_seconds);
}

int fv_hash_windows_device(fv_hasher* hs, const int32_t* d_idx, uint64_t nwin, uint32_t window, int weighted,
                           uint32_t hash_length, uint32_t flags, uint8_t* d_out, double* kernel_seconds) {
  FV_REQUIRE(hs && (nwin == 0 || (d_idx && d_out)), FV_ERR_INVALID, "fv_hash_windows_device: NULL argument");
  FV_REQUIRE(window >= 1 && window <= 32, FV_ERR_INVALID, "window must be in [1, 32], got %u", window);
  if (weighted) FV_REQUIRE(hs->h.f != nullptr, FV_ERR_STATE, "weighted window hashing needs an inverse frequency table");
  fv::DeviceGuard guard(hs->device);
  return run_hash(hs, weighted ? 1 : 2, d_idx, nwin, (int)window, hash_length, flags, d_out, kernel_seconds);
}

// Host-buffer forms.  The batch goes through the GPU in chunks on two pipeline slots (a stream with
// its own device buffers each), so the upload of one chunk, the kernel of the previous one and the
// download of the one before overlap; the buffers live as long as the hasher.  Page-locked caller
// memory (fv_host_alloc_pinned) is copied from and to directly; pageable memory is staged through
// the slots' pinned buffers by host threads while the GPU works on the other slot.
constexpr size_t PIPE_BYTES = (size_t)16 << 20;  // per buffer

static bool is_pinned(const void* p) {
  cudaPointerAttributes a;
  if (cudaPointerGetAttributes(&a, p) != cudaSuccess) {
    cudaGetLastError();
    return false;
  }
  return a.type == cudaMemoryTypeHost;
}
static void host_copy(void* dst, const void* src, size_t bytes) {
  constexpr size_t PART = (size_t)1 << 20;
  const long long parts = (long long)((bytes + PART - 1) / PART);
#pragma omp parallel for schedule(static) if (parts > 4)
  for (long long i = 0; i < parts; ++i) {
    const size_t o = (size_t)i * PART;
    memcpy(static_cast<char*>(dst) + o, static_cast<const char*>(src) + o, bytes - o < PART ? bytes - o : PART);
  }
}
static int ensure_pipeline(fv_hasher* hs) {
  if (hs->pipe_bytes) return FV_OK;
  for (int b = 0; b < 2; ++b) {
    FV_CUDA(cudaStreamCreateWithFlags(&hs->pipe_stream[b], cudaStreamNonBlocking));
    FV_CUDA(cudaEventCreateWithFlags(&hs->pipe_done[b], cudaEventDisableTiming));
    FV_CUDA(cudaMalloc((void**)&hs->pipe_d_in[b], PIPE_BYTES));
    FV_CUDA(cudaMalloc((void**)&hs->pipe_d_out[b], PIPE_BYTES));
    FV_CUDA(cudaHostAlloc((void**)&hs->pipe_h_in[b], PIPE_BYTES, cudaHostAllocDefault));
    FV_CUDA(cudaHostAlloc((void**)&hs->pipe_h_out[b], PIPE_BYTES, cudaHostAllocDefault));
  }
  hs->pipe_bytes = PIPE_BYTES;
  return FV_OK;
}

static int hash_host(fv_hasher* hs, int mode, const int32_t* in, uint64_t n, size_t in_per_item, uint32_t window,
                     uint32_t hash_length, uint32_t flags, uint8_t* out) {
  if (n == 0) return FV_OK;
  fv::DeviceGuard guard(hs->device);
  FV_REQUIRE(guard.ok, FV_ERR_CUDA, "cannot select device %d", hs->device);
  FV_TRY(ensure_pipeline(hs));
  const size_t out_per = (flags & FV_HASH_BYTES) ? (size_t)hs->h.K : (size_t)((hs->h.K + 7) / 8);
  const size_t in_bytes = in_per_item * sizeof(int32_t);
  // token batches much larger than the vocabulary: hash the vocabulary once, then every chunk gathers
  const bool table = (mode == 0 && n >= 4ull * (unsigned long long)hs->h.V);
  if (table) FV_TRY(run_hash_table(hs, nullptr, 0, hash_length, flags, nullptr, nullptr));
  FV_CUDA(cudaMemsetAsync(hs->d_err, 0, sizeof(uint32_t), hs->stream));
  FV_CUDA(cudaStreamSynchronize(hs->stream));
  const size_t per_max = in_bytes > out_per ? in_bytes : out_per;
  const uint64_t chunk = std::max<uint64_t>(PIPE_BYTES / per_max, 1);
  const bool in_direct = is_pinned(in), out_direct = is_pinned(out);
  uint64_t pending_first[2] = {0, 0}, pending_n[2] = {0, 0};  // chunk whose codes still sit in the slot's pinned buffer
  uint64_t c = 0;
  for (uint64_t first = 0; first < n; first += chunk, ++c) {
    const int b = (int)(c & 1);
    const uint64_t m = std::min<uint64_t>(chunk, n - first);
    if (c >= 2) {  // the slot's previous chunk must have left it
      FV_CUDA(cudaEventSynchronize(hs->pipe_done[b]));
      if (!out_direct) host_copy(out + pending_first[b] * out_per, hs->pipe_h_out[b], pending_n[b] * out_per);
    }
    const int32_t* src = in + first * in_per_item;
    if (!in_direct) {
      host_copy(hs->pipe_h_in[b], src, m * in_bytes);
      src = hs->pipe_h_in[b];
    }
    cudaStream_t st = hs->pipe_stream[b];
    FV_CUDA(cudaMemcpyAsync(hs->pipe_d_in[b], src, m * in_bytes, cudaMemcpyHostToDevice, st));
    if (table)
      enqueue_gather(hs, st, hs->pipe_d_in[b], m, (int)out_per, hs->pipe_d_out[b]);
    else
      enqueue_hash(hs, st, mode, hs->pipe_d_in[b], m, (int)window, hash_length, flags, hs->pipe_d_out[b]);
    FV_CUDA(cudaGetLastError());
    FV_CUDA(cudaMemcpyAsync(out_direct ? out + first * out_per : hs->pipe_h_out[b], hs->pipe_d_out[b], m * out_per,
                            cudaMemcpyDeviceToHost, st));
    FV_CUDA(cudaEventRecord(hs->pipe_done[b], st));
    pending_first[b] = first;
    pending_n[b] = m;
  }
  for (uint64_t k = (c >= 2 ? c - 2 : 0); k < c; ++k) {  // drain in order
    const int b = (int)(k & 1);
    FV_CUDA(cudaEventSynchronize(hs->pipe_done[b]));
    if (!out_direct) host_copy(out + pending_first[b] * out_per, hs->pipe_h_out[b], pending_n[b] * out_per);
  }
  uint32_t err = 0;
  FV_CUDA(cudaMemcpy(&err, hs->d_err, sizeof(err), cudaMemcpyDeviceToHost));
  if (err & FV_DEVERR_TOKEN_RANGE) return fv::fail(FV_ERR_DATA, "an input id was out of range (device check)");
  return FV_OK;
}

int fv_hash_tokens(fv_hasher* hs, const int32_t* ids, uint64_t n, uint32_t hash_length, uint32_t flags, uint8_t* out) {
  FV_REQUIRE(hs && (n == 0 || (ids && out)), FV_ERR_INVALID, "fv_hash_tokens: NULL argument");
  FV_REQUIRE(hash_length >= 1 && (int)hash_length < hs->h.K, FV_ERR_INVALID,
             "hash_length must be in [1, K-1] (K = %d), got %u", hs->h.K, hash_length);
  return hash_host(hs, 0, ids, n, 1, 0, hash_length, flags, out);
}

// ---------------------------------------------------------------------------
// Token hashing without any allocation.
//
// fv_hash_tokens makes its staging buffers (device memory, pinned host memory and, for large
// batches, a table of the whole vocabulary's codes) the first time it is called on a hasher.
// That is fine for bulk work, but two kinds of callers of this library cannot allocate at
// that moment: a process whose device memory is owned up front by somebody else's pool,
// where an extra cudaMalloc may simply fail, and a service that answers a few query tokens
// at a time beside a trainer that already fills the GPU and must not see its footprint grow.
// For them the staging area is the fixed array below: it is part of the library image, so
// every GPU that loads the library holds these FV_STATIC_SCRATCH_BYTES until the process
// exits, whether the call is used or not.
//
// The array's name is only a handle on the host; the device address is looked up
// once per device with cudaGetSymbolAddress (with that device current) the first
// time the entry point runs there.  Make that first call before starting any
// stream capture.  All calls share the one array and it keeps whatever the last
// call left in it: the ids are overwritten by the upload and the kernel writes every
// output byte that is copied back, so nothing in it has to be cleared (the error
// word the kernel reports through is reset before each launch).  Two calls that
// overlap on the same GPU -- different hashers, different host threads -- would
// race on the array; callers must serialise them.
// ---------------------------------------------------------------------------
#define FV_STATIC_SCRATCH_BYTES (8u << 20)
static __device__ __align__(256) unsigned char g_hash_scratch[FV_STATIC_SCRATCH_BYTES];
static void* g_hash_scratch_addr[64] = {nullptr};

int fv_hash_tokens_static(fv_hasher* hs, const int32_t* ids, uint64_t n, uint32_t hash_length, uint32_t flags,
                          uint8_t* out) {
  FV_REQUIRE(hs && (n == 0 || (ids && out)), FV_ERR_INVALID, "fv_hash_tokens_static: NULL argument");
  FV_REQUIRE(hash_length >= 1 && (int)hash_length < hs->h.K, FV_ERR_INVALID,
             "hash_length must be in [1, K-1] (K = %d), got %u", hs->h.K, hash_length);
  FV_REQUIRE(hs->device >= 0 && hs->device < 64, FV_ERR_INVALID, "device %d out of range", hs->device);
  if (n == 0) return FV_OK;
  const size_t out_per = (flags & FV_HASH_BYTES) ? (size_t)hs->h.K : (size_t)((hs->h.K + 7) / 8);
  const size_t per_item = sizeof(int32_t) + out_per;
  const size_t max_items = (FV_STATIC_SCRATCH_BYTES - 256) / per_item;
  FV_REQUIRE(n <= max_items, FV_ERR_INVALID,
             "fv_hash_tokens_static: %llu tokens need %llu bytes of staging, the fixed area holds %u bytes "
             "(at most %llu tokens for K = %d in this output format); split the batch or use fv_hash_tokens",
             (unsigned long long)n, (unsigned long long)(n * per_item + 256), FV_STATIC_SCRATCH_BYTES,
             (unsigned long long)max_items, hs->h.K);
  fv::DeviceGuard guard(hs->device);
  FV_REQUIRE(guard.ok, FV_ERR_CUDA, "cannot select device %d", hs->device);
  if (!g_hash_scratch_addr[hs->device]) {
    void* p = nullptr;
    FV_CUDA(cudaGetSymbolAddress(&p, g_hash_scratch));
    g_hash_scratch_addr[hs->device] = p;
  }
  unsigned char* base = static_cast<unsigned char*>(g_hash_scratch_addr[hs->device]);
  int32_t* d_ids = reinterpret_cast<int32_t*>(base);
  uint8_t* d_out = base + ((n * sizeof(int32_t) + 255) & ~(size_t)255);
  FV_CUDA(cudaMemcpyAsync(d_ids, ids, n * sizeof(int32_t), cudaMemcpyHostToDevice, hs->stream));
  const int rc = run_hash(hs, 0, d_ids, n, 0, hash_length, flags, d_out, nullptr, /*may_allocate=*/false);
  if (rc != FV_OK) {
    cudaStreamSynchronize(hs->stream);  // the upload must not outlive the caller's ids
    return rc;
  }
  FV_CUDA(cudaMemcpyAsync(out, d_out, n * out_per, cudaMemcpyDeviceToHost, hs->stream));
  FV_CUDA(cudaStreamSynchronize(hs->stream));
  return FV_OK;
}

int fv_hash_windows(fv_hasher* hs, const int32_t* idx, uint64_t nwin, uint32_t window, const float* inv_freq,
                    uint32_t hash_length, uint32_t flags, uint8_t* out) {
  FV_REQUIRE(hs && (nwin == 0 || (idx && out)), FV_ERR_INVALID, "fv_hash_windows: NULL argument");
  FV_REQUIRE(window >= 1 && window <= 32, FV_ERR_INVALID, "window must be in [1, 32], got %u", window);
  FV_REQUIRE(hash_length >= 1 && (int)hash_length < hs->h.K, FV_ERR_INVALID,
             "hash_length must be in [1, K-1] (K = %d), got %u", hs->h.K, hash_length);
  const bool raw = (flags & FV_HASH_RAW) || inv_freq == nullptr;
  if (!raw) FV_TRY(fv_hasher_set_inverse_frequency(hs, inv_freq, (uint32_t)hs->h.V));
  return hash_host(hs, raw ? 2 : 1, idx, nwin, window, window, hash_length, flags, out);
}

}  // extern "C"
