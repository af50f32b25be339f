// A small CUDA execution model for the host -- TEST INFRASTRUCTURE ONLY.
//
// It lets `__global__` functions written for nvcc be compiled by g++ and executed on
// the CPU with CUDA's semantics for the handful of features the reference's training
// kernels use: threadIdx/blockIdx/blockDim/gridDim, static and dynamic `__shared__`
// memory, `__syncthreads()`, `__shfl_down_sync()`, `atomicAdd(float*)` and `__ldg`.
//
// Execution model.  Blocks of a grid run one after the other (any block order is a
// valid CUDA schedule).  The threads of a block are cooperative fibers on one OS
// thread; a fiber runs until it finishes or reaches a synchronisation point:
//   * __syncthreads():  released once every live thread of the block waits there;
//   * __shfl_down_sync(): every lane posts its value, the warp meets, every lane
//     reads the value its source lane posted -- all 32 lanes exchange at the same
//     instant, as the hardware does.
// Fibers of a block are resumed in thread order, so floating-point atomics are applied
// in thread order within a block and block order within a grid: one admissible order of
// the hardware's.  Shared variables are `thread_local` objects of the one OS thread.
// Nothing in the product includes this header.
#pragma once

#include <math.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <cmath>
#include <functional>
#include <vector>

struct dim3 {
  unsigned x, y, z;
  dim3(unsigned x_ = 1, unsigned y_ = 1, unsigned z_ = 1) : x(x_), y(y_), z(z_) {}
};
typedef unsigned int uint;

// The built-in variables.  The scheduler sets threadIdx whenever it resumes a fiber.
extern thread_local dim3 threadIdx, blockIdx, blockDim, gridDim;

#define __global__ static
#define __device__
#define __host__
#define __shared__ thread_local
// dynamic shared memory: kernels declare `extern __shared__ char s[];`
constexpr size_t COH_DYN_SMEM = 64 * 1024;
extern thread_local char s[COH_DYN_SMEM];

namespace coh {

enum Wait { RUNNABLE = 0, AT_BLOCK = 1, AT_WARP = 2, DONE = 3 };

struct Fiber {
  void* sp = nullptr;  // saved stack pointer while switched out
  char* stack = nullptr;
  dim3 tid;
  int wait = DONE;
  int linear = 0;
};

struct Block {
  std::vector<Fiber> fibers;
  void* sched_sp = nullptr;
  Fiber* cur = nullptr;
  const std::function<void()>* body = nullptr;
  // shuffle mailboxes: [parity][thread]
  std::vector<unsigned long long> slot[2];
  std::vector<unsigned> shfl_count;  // shuffles executed so far, per thread
};
extern thread_local Block* g_blk;

// Context switch: saves the callee-saved registers on the current stack, stores the stack
// pointer in *from, loads `to` and restores.  (System V x86-64 ABI.)
extern "C" void coh_switch(void** from, void* to);

void yield_to_scheduler(int wait);
// may_sync = false: the kernel has no __syncthreads / shuffles, so its threads run as plain loops.
void launch(dim3 grid, dim3 block, size_t smem_bytes, const std::function<void()>& body, bool may_sync = true);

}  // namespace coh

inline void __syncthreads() { coh::yield_to_scheduler(coh::AT_BLOCK); }

template <typename T>
inline T __shfl_down_sync(unsigned /*mask*/, T v, unsigned delta, int width = 32) {
  static_assert(sizeof(T) <= 8, "shuffle payload");
  coh::Block* b = coh::g_blk;
  coh::Fiber* f = b->cur;
  const int me = f->linear;
  const unsigned par = b->shfl_count[me] & 1u;
  unsigned long long raw = 0;
  memcpy(&raw, &v, sizeof(T));
  b->slot[par][me] = raw;
  b->shfl_count[me] += 1;
  coh::yield_to_scheduler(coh::AT_WARP);  // every lane of the warp has posted
  const int lane = me & 31;
  const int seg_end = (lane / width) * width + width;  // first lane past this lane's segment
  const int src = (lane + (int)delta < seg_end) ? me + (int)delta : me;
  const int warp_last = (me | 31) < (int)b->fibers.size() ? (me | 31) : (int)b->fibers.size() - 1;
  const unsigned long long got = b->slot[par][src <= warp_last ? src : me];
  T out;
  memcpy(&out, &got, sizeof(T));
  return out;
}

template <typename T>
inline T __ldg(const T* p) {
  return *p;
}
inline float atomicAdd(float* p, float v) {
  const float old = *p;
  *p = old + v;
  return old;
}
