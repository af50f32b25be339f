// Scheduler of the CUDA-on-host execution model (see cuda_on_host.h) -- TEST INFRASTRUCTURE ONLY.
#include "cuda_on_host.h"

#if !defined(__x86_64__)
#error "cuda_on_host: the fiber switch is written for x86-64 (System V ABI)"
#endif

thread_local dim3 threadIdx, blockIdx, blockDim, gridDim;
alignas(64) thread_local char s[COH_DYN_SMEM];

asm(R"(
.text
.globl coh_switch
.type coh_switch,@function
coh_switch:
  pushq %rbp
  pushq %rbx
  pushq %r12
  pushq %r13
  pushq %r14
  pushq %r15
  movq %rsp, (%rdi)
  movq %rsi, %rsp
  popq %r15
  popq %r14
  popq %r13
  popq %r12
  popq %rbx
  popq %rbp
  ret
.size coh_switch,.-coh_switch
)");

namespace coh {

thread_local Block* g_blk = nullptr;
constexpr size_t STACK_BYTES = 48 * 1024;

static void fiber_entry() {
  Block* b = g_blk;
  (*b->body)();
  b->cur->wait = DONE;
  coh_switch(&b->cur->sp, b->sched_sp);
  abort();  // a finished fiber is never resumed
}

void yield_to_scheduler(int wait) {
  Block* b = g_blk;
  if (!b || !b->cur) {
    fprintf(stderr, "cuda_on_host: a kernel launched without fibers reached a synchronisation point\n");
    abort();
  }
  Fiber* f = b->cur;
  f->wait = wait;
  coh_switch(&f->sp, b->sched_sp);
}

static void prepare(Fiber& f) {
  uintptr_t top = (reinterpret_cast<uintptr_t>(f.stack) + STACK_BYTES) & ~(uintptr_t)15;
  void** p = reinterpret_cast<void**>(top);
  *--p = nullptr;                                    // where fiber_entry would return to (it never does)
  *--p = reinterpret_cast<void*>(&fiber_entry);      // popped by the `ret` of coh_switch
  for (int i = 0; i < 6; ++i) *--p = nullptr;        // rbp rbx r12 r13 r14 r15
  f.sp = p;
  f.wait = RUNNABLE;
}

void launch(dim3 grid, dim3 block, size_t smem_bytes, const std::function<void()>& body, bool may_sync) {
  if (smem_bytes > COH_DYN_SMEM) {
    fprintf(stderr, "cuda_on_host: %zu bytes of dynamic shared memory requested, %zu available\n", smem_bytes, COH_DYN_SMEM);
    abort();
  }
  const int T = (int)(block.x * block.y * block.z);
  gridDim = grid;
  blockDim = block;
  if (T == 1 || !may_sync) {
    // no thread of this kernel waits for another one: plain loops, thread order within block order
    // (a synchronisation point reached anyway aborts with a message)
    g_blk = nullptr;
    for (unsigned bz = 0; bz < grid.z; ++bz)
      for (unsigned by = 0; by < grid.y; ++by)
        for (unsigned bx = 0; bx < grid.x; ++bx) {
          blockIdx = dim3(bx, by, bz);
          for (unsigned tz = 0; tz < block.z; ++tz)
            for (unsigned ty = 0; ty < block.y; ++ty)
              for (unsigned tx = 0; tx < block.x; ++tx) {
                threadIdx = dim3(tx, ty, tz);
                body();
              }
        }
    return;
  }
  Block blk;
  blk.body = &body;
  blk.fibers.resize(T);
  blk.slot[0].assign(T, 0ull);
  blk.slot[1].assign(T, 0ull);
  blk.shfl_count.assign(T, 0u);
  char* stacks = static_cast<char*>(malloc((size_t)T * STACK_BYTES));
  if (!stacks) abort();
  for (int t = 0; t < T; ++t) {
    Fiber& f = blk.fibers[t];
    f.stack = stacks + (size_t)t * STACK_BYTES;
    f.linear = t;
    f.tid = dim3(t % block.x, (t / block.x) % block.y, t / (block.x * block.y));
  }
  g_blk = &blk;
  for (unsigned bz = 0; bz < grid.z; ++bz)
    for (unsigned by = 0; by < grid.y; ++by)
      for (unsigned bx = 0; bx < grid.x; ++bx) {
        blockIdx = dim3(bx, by, bz);
        for (int t = 0; t < T; ++t) {
          prepare(blk.fibers[t]);
          blk.shfl_count[t] = 0u;
        }
        for (;;) {
          bool ran = false;
          for (int t = 0; t < T; ++t) {
            Fiber& f = blk.fibers[t];
            if (f.wait != RUNNABLE) continue;
            threadIdx = f.tid;
            blk.cur = &f;
            coh_switch(&blk.sched_sp, f.sp);
            ran = true;
          }
          blk.cur = nullptr;
          // release the meeting points that are complete
          int live = 0, at_block = 0;
          for (int t = 0; t < T; ++t) {
            live += blk.fibers[t].wait != DONE;
            at_block += blk.fibers[t].wait == AT_BLOCK;
          }
          if (live == 0) break;
          bool released = false;
          if (at_block == live) {
            for (int t = 0; t < T; ++t)
              if (blk.fibers[t].wait == AT_BLOCK) blk.fibers[t].wait = RUNNABLE;
            released = true;
          }
          for (int w0 = 0; w0 < T; w0 += 32) {
            int wl = 0, ww = 0;
            for (int t = w0; t < T && t < w0 + 32; ++t) {
              wl += blk.fibers[t].wait != DONE;
              ww += blk.fibers[t].wait == AT_WARP;
            }
            if (wl > 0 && ww == wl) {
              for (int t = w0; t < T && t < w0 + 32; ++t)
                if (blk.fibers[t].wait == AT_WARP) blk.fibers[t].wait = RUNNABLE;
              released = true;
            }
          }
          (void)ran;
          if (!released) {
            fprintf(stderr, "cuda_on_host: deadlock in block (%u,%u,%u): its threads wait at different points\n", bx, by, bz);
            abort();
          }
        }
      }
  g_blk = nullptr;
  free(stacks);
}

}  // namespace coh
