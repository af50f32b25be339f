// FlyVec trainer for sm_100a: one handle = one GPU = one data-parallel rank.
//
// Data layout in HBM
//   wt      float [N][Kp]   transposed synapses: row i holds the Kp (K padded to a
//                           multiple of 4) weights of input i, so the activation of
//                           a window is a sum of w contiguous rows.
//   alpha   double[2][Kp]   per-unit scale; the synapse matrix is alpha[mu]*wt[i][mu].
//                           The dense part of the Hebbian update, W_mu *= (1 - s*X_mu),
//                           only touches alpha; wt changes at the scattered positions.
//   tokens, wstart, perm    corpus, window starts, window order.
//   idx     int  [32][G*B][w] input ids of the next steps (all ranks' windows), two staging buffers.
//   mailbox                 per rank and step parity a packet of 64-bit words {payload, step sequence
//                           number}: B winners, (with delta) B second winners, Kp floats of xx.
//   xx_hi/lo  u64 [8][Kp]   fixed-point accumulators of xx; rec/cnt [G*B*w + 64*Kp] scatter bookkeeping: one
//                           record per distinct touched position.
//   hot_cnt u32 [64][Kp]    requests per (row of one of the 32 most frequent tokens, unit) pair, counted by
//                           k_forward; with several ranks the counts travel in a "hotbox" beside the packets.
//
// One global step (reference: run_epoch, flyvec/src/cuda_funcs.cu:1662-1812):
//   (k_build_idx_block, on a side stream: T4, ids of the next 32 steps   (cuda_funcs.cu:915-936))
//   k_forward    T6-8 gather-sum, arg-max, weighted winner    (cuda_funcs.cu:248-305, 488-561)
//                T8   every window adds its term of xx[mu] as a fixed-point number: the sum does not
//                     depend on the order of arrival          (cuda_funcs.cu:722-744)
//   k_tag        T10  each touched (mu,i) gets one owner record; its weight is parked there and
//                     replaced by a tagged NaN                 (cuda_funcs.cu:657-672); requests for hot
//                     pairs are not claimed one by one: one thread per pair claims the counted total
//                     (k_tag_batch: the same with several slots per thread, for steps of several ranks);
//                     its first CTA turns the xx sums into floats (xx_finish); with several ranks
//                     eight more CTAs copy this rank's winners into the peers' mailboxes, and every
//                     consumer of a peer's word checks the sequence number the word carries
//                     (or, without peer access: k_xx, then one NCCL all-gather of the packets)
//   k_update     T11  nc = max|D|: exact D at touched positions; the largest |wt| over untouched ones
//                     from per-unit candidate rows kept from step to step, no pass over the matrix
//                                                              (cu_special_reduction.cu:26-99)
//                T12-13 s = eps/max(prec,nc); alpha *= 1 - s*X; touched weights restored plus their
//                     scatter term                             (cuda_funcs.cu:1797-1799,
//                                                               cu_special_reduction.cu:316-354)
//                     (= k_eval + k_apply in one launch; the step after new weights or a fold runs them
//                     apart with k_colscan and k_collect, which rebuild the candidate rows, in between;
//                     k_scan is the every-step matrix pass the candidate rows replace)
#include <dlfcn.h>

#include <algorithm>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

#include "fv_common.h"

namespace {

constexpr unsigned FULL = 0xffffffffu;
constexpr uint32_t TAG_BASE = 0x7f800000u;  // exponent all ones: tag = TAG_BASE | (slot+1)
constexpr uint32_t ABS_MASK = 0x7fffffffu;
constexpr int MAX_K = 1024;

constexpr int XX_SLOTS = 8;  // copies of the xx accumulators (spread by window index)
struct StepCtl {
  unsigned long long base;  // schedule index of the step launched with local == 0
  unsigned long long tick;  // steps executed since the weights were last folded (selects the alpha buffer)
  float eps;
  float delta;            // anti-Hebbian strength of the running epoch (cuda_funcs.cu:1230)
  uint32_t error;
  uint32_t wabsmax;       // bit pattern of an upper bound of max |wt|
  uint32_t wabsmax_fold;  // the same, collected while folding
  int32_t xx_kexp;        // xx is accumulated in units of 2^-xx_kexp this step (written by k_forward)
  uint32_t fwd_next[2];   // window tickets k_forward hands out beyond the first round, by step parity
  uint32_t scan_ticket;   // CTAs of the running k_scan that have finished
  uint32_t apply_ticket;  // (unused)
  uint32_t out_count;     // (unused)
  uint32_t pad;
  uint32_t list_count[2]; // records reserved in this step's touched-position list, by step parity
  unsigned long long update_arrivals;  // CTAs of k_update that have reached the meeting point, over all steps
  uint32_t need_scan;     // (unused)
  uint32_t scans_run;     // units whose column k_eval had to read in this call (their candidates were all touched)
  // Device-side phase clock: every step kernel's first thread charges the time since the previous
  // mark to the phase that was running and names its own.  No events, so the launches stay chained.
  unsigned long long t_mark;
  unsigned long long phase_ns[8];
  uint32_t phase_now;
  uint32_t pad2;
};
enum Phase { PH_OTHER = 0, PH_FORWARD = 1, PH_XX = 2, PH_WAIT = 3, PH_TAG = 4, PH_SCAN = 5, PH_APPLY = 6, PH_FOLD = 7 };

// Everything a kernel needs, passed by value.
constexpr int HOT_TOKENS = 32;            // most frequent tokens whose two rows (context, target) are hot
constexpr int HOT_ROWS = 2 * HOT_TOKENS;

struct Dev {
  int K, Kp, Kq, V, N, W, B, G, rank, P, XO;  // P = packet words, XO = offset of xx inside a packet
  // Steps this trainer had executed when the running call began.  A kernel's step number is tick0 + local:
  // the host knows it, so no kernel has to fetch it from the control block before it can form an address.
  unsigned long long tick0;
  // exact n / divisor for n < 2^31 as (n * m) >> s (64-bit product): m = ceil(2^s / divisor), s = 31 + ceil(log2 divisor)
  uint32_t mW, sW, mB, sB, mKp, sKp, mG, sG;
  int idx_rstride; // ids of a step: rank r's block of B*W ids starts r * idx_rstride elements into the step's buffer
  int MO;          // offset of the second winners inside a packet (only with delta != 0)
  int has_delta;   // the anti-Hebbian term is on: every window also names its m-th (second) winner
  unsigned long long Ns, ntok;
  float prec;
  uint32_t flags;
  float* wt;
  double* alpha;
  const int32_t* tokens;
  const unsigned long long* wstart;
  const unsigned long long* perm;
  const float* f;
  uint32_t* mail;          // this rank's mailbox: MAIL_HDR words of flags, then packets [2][G][P]
  uint32_t* const* peers;  // device table of all ranks' mailboxes (peer-mapped), or null
  unsigned spin_limit;     // polls before a wait on a peer's flag gives up
  int shard;               // 1: rows i with i % G == rank are tagged and scanned here; every other row's scatter
                           // counts arrive from its owner (see the inbox below)
  size_t inbox_off;        // word offset of the inbox [G][G*B*W] of 64-bit update entries inside the mailbox
  size_t inbox_cap;        // entries per sender
  // xx accumulators [XX_SLOTS][Kp]: fixed-point sums (high and low 32-bit digits, each in a 64-bit word) and the
  // number of windows won; filled by k_forward, turned into floats and cleared by xx_finish
  unsigned long long* xx_hi;
  unsigned long long* xx_lo;
  uint32_t* xx_wins;
  float fmax;      // upper bound of the inverse frequencies (scales the fixed-point unit)
  int32_t* cnt;    // per record: later comers that add +f_i (first winner's row)
  int32_t* cntn;   // per record: later comers that add -delta*f_i (second winner's row); null without delta
  uint4* rec;      // [rec_cap] touched-position records {position, parked weight bits, 1/count bits, multiplicities}
  int rec_cap;     // records the list can hold: every (window, position) of a step plus one per hot pair
  // Hot rows: the rows of the most frequent tokens.  A (hot row, unit) pair is asked for by hundreds of windows
  // of a step; claimed one by one, those requests queue at one L2 address.  Instead k_forward counts them per
  // pair as it finds the winners (fire-and-forget reductions spread over the whole pass) and the tagging kernel
  // claims every non-empty pair once, with its count.  Which rows are "hot" never changes a result.
  int nhot;                  // hot rows in use by the running step loop (0: off)
  const int8_t* hotidx;      // [N+1] hot-row number of a matrix row, or -1
  const int32_t* hot_rows;   // [nhot] matrix row of a hot-row number
  uint32_t* hot_cnt;         // [HOT_ROWS][Kp] windows that want +f_i at (hot row, unit); zero between steps
  uint32_t* hot_cntn;        // the same for the second winner's -delta*f_i; null without delta
  int hot_x;                 // several ranks with peer mailboxes: the counts of all ranks travel (hotbox), so that
                             // every hot-row slot of every rank is skipped; else a rank counts what its own forward pass saw
  size_t hot_off;            // word offset of the hotbox inside the mailbox: u64 [2][G][HC] flagged count words
  int HC;                    // count words per rank and step: HOT_ROWS * Kp, twice that with delta
  uint32_t* colmax;
  uint32_t* ncb;
  // Candidate rows of the column maxima (see k_eval): per unit up to CAND_CAP rows and a floor that bounds
  // |wt| of every scanned row outside the list.
  int use_cand;
  int32_t* cand_rows;             // [Kp][CAND_CAP]
  int32_t* cand_n;                // [Kp] rows listed (may count past CAND_CAP: clamp)
  uint32_t* cand_floor;           // [Kp] bit pattern of the floor
  uint32_t* cand_unc;             // [Kp] 1: the running step could not certify this unit's maximum from its list
  unsigned long long* colarg;     // [Kp] (bit pattern << 32 | row) of the column maximum found by k_colscan
  double* stat_x;  // [2][Kp] mean xx over the active ranks, written by the scan for the apply kernel
  int32_t* stat_n; // [2][Kp] number of active ranks
  StepCtl* ctl;
  float* nc_log;
  float* s_log;
};

// Mailbox header (32-bit words).  Everything is indexed [parity][sender]; a flag holds the sequence
// number (tick + local + 1) of the step whose data is complete.
constexpr int MAX_RANKS = 16;
// The partial normaliser and the length of a rank's entry list travel inside their flag: one 64-bit word
// (sequence number in the high half, payload in the low half) written with a single store.
constexpr int WORD_NC = 2 * MAX_RANKS;         // u64 [2][MAX_RANKS]: seq | float bits of sender's partial nc
constexpr int WORD_OUT = 6 * MAX_RANKS;        // u64 [2][MAX_RANKS]: seq | records in sender's touched-position list
constexpr int MAIL_HDR = 512;                  // words; keeps the packets 2 KiB aligned
// Packet of rank r for the step of the given parity: P 64-bit words -- B winners, (with delta) B
// second winners at MO, Kp floats of xx at XO.  Every word carries its own flag: payload in the low
// half, the step's sequence number in the high half, written with ONE 8-byte store, which arrives
// whole.  A producer therefore stores a word straight into every peer's copy of its packet the
// moment the value exists and never fences; a consumer reads the word and knows from the sequence
// number whether it is this step's.
__device__ __forceinline__ unsigned long long* packet(const Dev& d, int parity, int r) {
  return reinterpret_cast<unsigned long long*>(d.mail + MAIL_HDR) + ((size_t)parity * d.G + r) * d.P;
}
__device__ __forceinline__ unsigned long long* peer_packet(const Dev& d, int peer, int parity, int r) {
  return reinterpret_cast<unsigned long long*>(d.peers[peer] + MAIL_HDR) + ((size_t)parity * d.G + r) * d.P;
}
__device__ __forceinline__ unsigned long long pk_word(uint32_t payload, uint32_t seq) {
  return ((unsigned long long)seq << 32) | payload;
}

// Sharded update.  Rank r owns the matrix rows i with i % G == r: it alone tags them, knows how often
// each of their positions was asked for and evaluates D there.  The other replicas need the same
// counts to move their copies: the owner stores one 64-bit entry per record of its touched-position
// list -- low half: position | ENTRY_VALID (or ENTRY_HOLE for a reserved record nobody claimed), high
// half: the count -- into every peer's inbox at [owner][record index], one 8-byte store that arrives
// whole.  A receiver takes entries [0, n) of a sender once it has the sender's record count n, waits
// (bounded) for an entry that is not there yet, applies it and clears it, so an entry is non-zero only
// between its arrival and its use.  A sender cannot write the entries of the next step before the
// receiver has used this step's: it needs the receiver's next winners first, and those leave after
// the receiver's update has finished.
constexpr uint32_t ENTRY_VALID = 0x80000000u;
constexpr uint32_t ENTRY_HOLE = 0xffffffffu;
__device__ __forceinline__ unsigned long long* inbox(const Dev& d, const uint32_t* mail, int sender) {
  return reinterpret_cast<unsigned long long*>(const_cast<uint32_t*>(mail) + d.inbox_off) + (size_t)sender * d.inbox_cap;
}
// Hot-pair counts of `sender` for the step of the given parity inside mailbox `mail`: HC flagged words.
__device__ __forceinline__ unsigned long long* hotbox(const Dev& d, const uint32_t* mail, int parity, int sender) {
  return reinterpret_cast<unsigned long long*>(const_cast<uint32_t*>(mail) + d.hot_off) + ((size_t)parity * d.G + sender) * d.HC;
}
__device__ __forceinline__ uint32_t fdiv(uint32_t n, uint32_t m, uint32_t s) {
  return (uint32_t)(((unsigned long long)n * m) >> s);
}
// Input id of slot e = (rank, window, position) of a step whose ranks' blocks lie idx_rstride apart.
__device__ __forceinline__ int step_id(const Dev& d, const int32_t* __restrict__ idx, int e) {
  const uint32_t r = fdiv(fdiv((uint32_t)e, d.mW, d.sW), d.mB, d.sB);
  return idx[(size_t)e + (size_t)r * (size_t)(d.idx_rstride - d.B * d.W)];
}
__device__ __forceinline__ unsigned long long global_timer() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ void phase_mark(StepCtl* c, uint32_t next) {
  const unsigned long long now = global_timer();
  c->phase_ns[c->phase_now & 7u] += now - c->t_mark;
  c->t_mark = now;
  c->phase_now = next;
}
// Message passing between GPUs: every word carries its own flag (a sequence number or a valid bit) and
// is written with ONE relaxed 8-byte store, which arrives whole; a consumer polls the word with relaxed
// loads (served by the local L2, where a peer's store over NVLink lands).  No fences.
__device__ __forceinline__ void store_relaxed_sys64(unsigned long long* p, unsigned long long v) {
  asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ void push_entry(const Dev& d, int k, uint32_t lo, int count) {
  const unsigned long long e = ((unsigned long long)(uint32_t)count << 32) | lo;
  for (int r = 0; r < d.G; ++r)
    if (r != d.rank) store_relaxed_sys64(inbox(d, d.peers[r], d.rank) + k, e);
}
__device__ __forceinline__ unsigned long long load_relaxed_sys64(const unsigned long long* p) {
  unsigned long long v;
  asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ bool wait_expired(const Dev& d, unsigned& polls) {
  if (++polls > d.spin_limit || (*reinterpret_cast<volatile uint32_t*>(&d.ctl->error) & FV_DEVERR_TIMEOUT)) {
    atomicOr(&d.ctl->error, FV_DEVERR_TIMEOUT);
    return true;
  }
  if (polls > 64) __nanosleep(128);
  return false;
}
// Bounded waits: they return false (and raise FV_DEVERR_TIMEOUT) when the limit is reached or another
// wait already failed; no wait in this library spins without a limit.
// Bounded wait for a {seq, payload} word; the payload needs no further ordering.
__device__ __forceinline__ bool wait_word(const Dev& d, const unsigned long long* word, uint32_t seq, uint32_t* payload) {
  unsigned polls = 0;
  for (;;) {
    const unsigned long long v = load_relaxed_sys64(word);
    if ((uint32_t)(v >> 32) == seq) {
      *payload = (uint32_t)v;
      return true;
    }
    if (wait_expired(d, polls)) return false;
  }
}

// Payload of a packet word once it carries the step's sequence number (bounded wait; `fallback`
// after a timeout, which also raises FV_DEVERR_TIMEOUT).  Words of this rank, and all words when
// the packets travel by all-gather, are complete before the reading kernel starts.
__device__ __forceinline__ uint32_t pk_read(const Dev& d, const unsigned long long* word, uint32_t seq, uint32_t fallback) {
  uint32_t payload = fallback;
  if (!wait_word(d, word, seq, &payload)) return fallback;
  return payload;
}

// Programmatic dependent launch: a kernel launched with the stream-serialization
// attribute may start while its predecessor in the stream is still draining; it must
// not touch anything the predecessor writes before this wait returns (the wait ends
// when the predecessor grid has completed and its memory is visible).
__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
// (An explicit early griddepcontrol.launch_dependents made the step slower on B200 --
// resident-but-waiting CTAs of the next kernel take slots from the running one -- so
// the dependents start at the implicit trigger, when this grid's CTAs exit.)

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o >= 1; o >>= 1) v = fmaxf(v, __shfl_xor_sync(FULL, v, o));
  return v;
}
__device__ __forceinline__ uint32_t warp_max_u32(uint32_t v) { return __reduce_max_sync(FULL, v); }

// ---------------------------------------------------------------------------
// control word
// ---------------------------------------------------------------------------
__global__ void k_set_ctl(StepCtl* ctl, unsigned long long base, float eps, float delta) {
  ctl->base = base;
  ctl->eps = eps;
  ctl->delta = delta;
  ctl->fwd_next[0] = ctl->fwd_next[1] = 0u;
  ctl->scans_run = 0u;
  for (int i = 0; i < 8; ++i) ctl->phase_ns[i] = 0ull;
  ctl->t_mark = global_timer();
  ctl->phase_now = PH_OTHER;
}
__global__ void k_reset_phase_clock(StepCtl* ctl) {
  for (int i = 0; i < 8; ++i) ctl->phase_ns[i] = 0ull;
  ctl->t_mark = global_timer();
  ctl->phase_now = PH_OTHER;
}
__global__ void k_advance(StepCtl* ctl, unsigned long long n) {
  grid_dependency_wait();
  phase_mark(ctl, PH_OTHER);
  ctl->base += n;
  ctl->tick += n;
}

// ---------------------------------------------------------------------------
// T4: input ids of every window of the global step (all ranks' blocks).
// Absent windows (past the end of the order) are marked -2 in every position.
// ---------------------------------------------------------------------------
__device__ __forceinline__ int input_id(const Dev& d, unsigned long long step, int e) {
  const int q = e / d.W, c = e - q * d.W;
  const unsigned long long pos = step * (unsigned long long)d.G * d.B + q;
  int val = -2;
  if (pos < d.Ns) {
    const unsigned long long p = d.perm[pos];
    if (p >= d.Ns) {
      atomicOr(&d.ctl->error, FV_DEVERR_WINDOW_RANGE);
    } else {
      const unsigned long long s = d.wstart[p];
      if (s + d.W > d.ntok) {
        atomicOr(&d.ctl->error, FV_DEVERR_WINDOW_RANGE);
      } else {
        const int tok = d.tokens[s + c];
        if (tok < 0) {
          val = -1;
        } else if (tok >= d.V) {
          atomicOr(&d.ctl->error, FV_DEVERR_TOKEN_RANGE);
          val = -1;
        } else {
          val = tok + (c == d.W / 2 ? d.V : 0);
        }
      }
    }
  }
  return val;
}
// Ids of `nsteps` consecutive global steps starting at `step0`, written back to back.  Runs on a
// side stream a block of steps ahead of the step loop: the ids depend on the corpus and the window
// order only, so the three dependent loads per id stay off the step's critical path.
__global__ void __launch_bounds__(256) k_build_idx_block(Dev d, unsigned long long step0, int nsteps,
                                                         int32_t* __restrict__ out) {
  const size_t per_step = (size_t)d.G * d.B * d.W;
  const size_t total = per_step * nsteps;
  for (size_t t = (size_t)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += (size_t)gridDim.x * blockDim.x) {
    const size_t s = t / per_step;
    out[t] = input_id(d, step0 + s, (int)(t - s * per_step));
  }
}

// Checks host-supplied input ids (streaming mode) against [ -2, N ); an id outside is reported and
// replaced by padding, so that no later kernel forms an address from it.
__global__ void k_check_idx(Dev d, int32_t* __restrict__ idx, size_t total) {
  grid_dependency_wait();
  for (size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += (size_t)gridDim.x * blockDim.x) {
    const int v = idx[e];
    if (v >= d.N || v < -2) {
      atomicOr(&d.ctl->error, FV_DEVERR_TOKEN_RANGE);
      idx[e] = -1;
    }
  }
}

// ---------------------------------------------------------------------------
// Forward pass.  One warp per window; lane l owns the float4 column groups
// l, l+32, ... of a row.  The winner is selected on the raw (unweighted)
// activation, the Hebbian coefficient uses the 1/count-weighted one
// (cuda_funcs.cu:1716-1721).
//
// Arithmetic.  The reference sums each unit in double over c = 0..w-1 and rounds
// to float (cuda_funcs.cu:252-260).  The fast path sums in float; sequential float
// summation of w terms bounded by xmax is off by at most w*w*2^-24*xmax, and the
// control word carries an upper bound of max |wt| (set when weights are loaded or
// folded, raised by k_apply), so when the gap between the two largest activations
// exceeds four times that bound (plus the rounding of the scale product) the
// arg-max of the float sums is the arg-max of the exact sums.
// Otherwise -- about one window in 10^4 -- the warp redoes the window in double
// with the reference's tie order.  Its kernel runs 64 threads per window: thread t
// keeps the lowest index of units t, t+64, ... (strict '>', cuda_funcs.cu:507-512);
// the __shfl_down_sync tree with offsets 16..1 and a strict '>' keeps the lower lane
// at every level (515-522), so among tied lanes the one with the smallest
// bit-reversed lane number reaches lane 0; thread 0 prefers warp 0 over warp 1
// (535-540).  Key among equal maxima: smallest (t / 32, bitreverse5(t % 32), index)
// with t = index % 64.
// ---------------------------------------------------------------------------
__device__ __forceinline__ int tie_key(int i) {
  const unsigned t = (unsigned)i & 63u;
  return (int)((((t & 32u) | (__brev(t & 31u) >> 27)) << 20) | (unsigned)i);
}
__device__ __forceinline__ bool better(float a, int ia, float b, int ib) {
  // true when (a, ia) beats (b, ib) under the reference's tie order
  if (a > b) return true;
  if (a < b) return false;
  return tie_key(ia) < tie_key(ib);
}

// The double-precision path for one window: per column group all w rows are fetched
// together (they were just read, so they come from L1/L2), summed in position order
// in double, scaled, rounded to float and compared with the reference's tie order.
// `skip` excludes one unit (used for the m-th winner).
__device__ __noinline__ int exact_winner(const float* __restrict__ wt, const double* __restrict__ alpha, int Kp, int Kq,
                                         int K, int W, int zrow, int my, int lane, int skip) {
  float best = -INFINITY;
  int bi = 0x000fffff;
  const int row_id = (my < 0) ? zrow : my;
  const int groups = (Kq + 31) >> 5;
  for (int t = 0; t < groups; ++t) {
    const int q = min(lane + 32 * t, Kq - 1);
    double s0 = 0, s1 = 0, s2 = 0, s3 = 0;
    for (int c0 = 0; c0 < W; c0 += 8) {
      float4 v[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const int id = __shfl_sync(FULL, row_id, (c0 + u) & 31);
        v[u] = __ldg(reinterpret_cast<const float4*>(wt + (size_t)((c0 + u < W) ? id : zrow) * Kp) + q);
      }
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        s0 += (double)v[u].x;
        s1 += (double)v[u].y;
        s2 += (double)v[u].z;
        s3 += (double)v[u].w;
      }
    }
    if (lane + 32 * t < Kq) {
      const int mu = 4 * q;
      const double s[4] = {s0, s1, s2, s3};
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        if (mu + k < K && mu + k != skip) {
          const float a = (float)(s[k] * alpha[mu + k]);
          if (better(a, mu + k, best, bi)) {
            best = a;
            bi = mu + k;
          }
        }
      }
    }
  }
#pragma unroll
  for (int o = 16; o >= 1; o >>= 1) {
    const float ob = __shfl_xor_sync(FULL, best, o);
    const int oi = __shfl_xor_sync(FULL, bi, o);
    if (better(ob, oi, best, bi)) {
      best = ob;
      bi = oi;
    }
  }
  return bi;
}

constexpr int FWD_THREADS = 128;
constexpr int FWD_WARPS = FWD_THREADS / 32;

// Two floats per 64-bit register; Blackwell adds both halves in one instruction.
__device__ __forceinline__ void add2(unsigned long long& a, const unsigned long long b) {
  asm("add.rn.f32x2 %0, %0, %1;" : "+l"(a) : "l"(b));
}
__device__ __forceinline__ float lo_f(unsigned long long v) { return __uint_as_float((unsigned)(v & 0xffffffffull)); }
__device__ __forceinline__ float hi_f(unsigned long long v) { return __uint_as_float((unsigned)(v >> 32)); }

// Weighted activation of the winner: float product with 1/count, double running sum
// over c = 0..w-1, float store (cuda_funcs.cu:289-305 restricted to one unit).
__device__ __forceinline__ float weighted_activation(const Dev& d, const double* __restrict__ alpha, int my, int winner,
                                                     int lane) {
  float x = 0.f;  // padding positions contribute +0, which leaves the double sum unchanged
  if (lane < d.W && my >= 0) {
    const float wv = (float)((double)d.wt[(size_t)my * d.Kp + winner] * alpha[winner]);
    x = wv * __ldg(d.f + (my % d.V));
  }
  double s = 0.0;
  for (int c = 0; c < d.W; ++c) s += (double)__shfl_sync(FULL, x, c);
  return (float)s;
}

// One warp per window.  The first nwarps windows are dealt statically, the rest is
// handed out through a counter in the control word, one window per request, so no
// warp idles while others still have a queue; outputs are keyed by window index, so
// the schedule does not influence any result.
//   * rows are gathered four at a time (two at a time for K > 640: 16 independent 128-bit loads per lane) and
//     added in position order with packed float adds (measured inside the step loop at
//     K=400, w=11: four rows, 128 registers, 16 warps per SM: 24.5 us; six rows, 166
//     registers, 12 warps: 25.6 us; the whole window, 221 registers, 8 warps: 28.3 us;
//     three rows, 96 registers, 20 warps: 26.4 us; two rows, 80 registers, 24 warps: 25.7 us;
//     requesting the next window's first rows ahead of the arg-max: 30.6 us with 168
//     registers, 31.6 us held to 128 with spills -- warps, not depth, hide the tail); padding positions gather an
//     all-zero row behind the matrix; lanes past the end of a row re-read its last
//     16 bytes instead of being predicated off.
//   * the float arg-max is certified when no other unit comes within theta of the
//     maximum; otherwise the window is redone in double on the spot.
template <int NT>
__global__ void __launch_bounds__(FWD_THREADS) k_forward(Dev d, int local, const int32_t* __restrict__ idx) {
  grid_dependency_wait();
  if (blockIdx.x == 0 && threadIdx.x == 0) phase_mark(d.ctl, PH_FORWARD);
  if (d.ctl->error & FV_DEVERR_TIMEOUT) return;  // a peer never answered: the step loop is void
  extern __shared__ __align__(16) unsigned char fwd_smem[];
  float* s_alpha = reinterpret_cast<float*>(fwd_smem);  // [Kp] the units' scales as floats

  const int lane = threadIdx.x & 31;
  const int warp = blockIdx.x * FWD_WARPS + (threadIdx.x >> 5);
  const int nwarps = gridDim.x * FWD_WARPS;
  const double* __restrict__ alpha = d.alpha + ((d.tick0 + local) & 1) * d.Kp;
  const int Kq = d.Kq;
  const int32_t* __restrict__ idx_own = idx + (size_t)d.rank * d.idx_rstride;

  // tickets: this launch draws from the counter of its parity and clears the other one, so that
  // consecutive launches need nobody else to reset anything
  const int par = (int)((d.tick0 + local) & 1);
  if (blockIdx.x == 0 && threadIdx.x == 0) d.ctl->fwd_next[par ^ 1] = 0u;

  int j = warp;
  int my = (j < d.B && lane < d.W) ? idx_own[(size_t)j * d.W + lane] : -1;

  float amax = 0.f;
  for (int mu = threadIdx.x; mu < d.Kp; mu += FWD_THREADS) s_alpha[mu] = (mu < d.K) ? (float)alpha[mu] : 0.f;
  for (int mu = lane; mu < d.K; mu += 32) amax = fmaxf(amax, fabsf((float)alpha[mu]));
  __syncthreads();
  amax = warp_max(amax);
  // Gap that certifies the float arg-max: 4 x (summation error w*w*u*xmax + scale rounding), u = 2^-24,
  // with xmax replaced by the bound on |alpha * wt| kept in the control word.
  const float theta = 4.0f * (float)(d.W * d.W + 2 * d.W + 4) * 5.9604645e-8f * amax * __uint_as_float(d.ctl->wabsmax);
  const bool force64 = (d.flags & FV_FLAG_ACC_FP64) != 0;
  // xx[mu] = sum of the winners' weighted activations (cuda_funcs.cu:722-744 adds them with float
  // atomics in arbitrary order).  Here every window adds its term as a fixed-point number in units
  // of 2^-kexp, two 32-bit digits in two 64-bit accumulators: integer addition commutes, so the sum
  // does not depend on the order the windows finish in and repeats from run to run, and it is
  // exact to 2^-32 of the unit.  The unit comes from a bound on any term,
  // |term| <= max|alpha| * max|wt| * w * max f * max(1, |delta|), so that 2*B terms cannot overflow.
  __shared__ int s_kexp;
  if (threadIdx.x == 0) {
    const double bound = (double)amax * (double)__uint_as_float(d.ctl->wabsmax) * (double)d.W * (double)d.fmax *
                         fmax(1.0, fabs((double)d.ctl->delta)) * 2.0 * (double)d.B;
    int e = (bound > 0.0 && bound < 1e300) ? ilogb(bound) + 1 : 0;  // bound < 2^e
    e = max(-200, min(e, 200));
    s_kexp = 92 - e;
    if (blockIdx.x == 0) d.ctl->xx_kexp = 92 - e;
  }
  __syncthreads();
  const int kexp = s_kexp;
  // term * 2^kexp as an integer (round to nearest), split at 2^32 with the low digit in [0, 2^32):
  // |term| = m * 2^(E - 150) with the 24-bit m of the float, so the product is m shifted by E - 150 + kexp
  auto xx_add = [&](int mu, float term, int j) {
    const uint32_t bits = __float_as_uint(term);
    const int E = (int)((bits >> 23) & 0xffu);
    const unsigned long long m = (bits & 0x007fffffu) | (E ? 0x00800000u : 0u);
    const int sh = (E ? E : 1) - 150 + kexp;
    unsigned long long hi = 0ull, lo = 0ull;  // |product| = hi * 2^32 + lo
    if (sh >= 32) {
      hi = (sh < 32 + 40) ? (m << (sh - 32)) : 0ull;  // m < 2^24 and the bound keep the product below 2^93
    } else if (sh >= 0) {
      const unsigned long long v = m << sh;  // < 2^56
      hi = v >> 32;
      lo = v & 0xffffffffull;
    } else if (sh > -25) {
      lo = (m + (1ull << (-sh - 1))) >> (-sh);
    }
    if (bits >> 31) {  // negative: floor at the split keeps the low digit non-negative
      hi = lo ? ~hi : (0ull - hi);
      lo = lo ? (0x100000000ull - lo) : 0ull;
    }
    // a popular unit wins hundreds of windows per step: XX_SLOTS copies of the accumulators, chosen
    // by the window index, keep the reductions from queueing on one address
    const int at = (j & (XX_SLOTS - 1)) * d.Kp + mu;
    if (hi) atomicAdd(d.xx_hi + at, hi);
    if (lo) atomicAdd(d.xx_lo + at, lo);
    d.xx_wins[mu] = 1u;  // "won a window": the same value from everybody, a plain store will do
  };

  // winners go into this rank's packet as flagged words; the tagging kernel forwards them to the peers.
  // (Storing them into the peers' memory from here, window by window, was measured on two GPUs: the
  // remote stores have to drain before this kernel can end -- 29.4 instead of 25.5 us -- and the tagging
  // kernel only gets 2.4 us shorter.)
  const uint32_t seq = (uint32_t)(d.tick0 + local + 1);
  unsigned long long* win_out = (lane == 0) ? packet(d, par, d.rank) : nullptr;
  const int zrow = d.N;  // the all-zero row
  // rows whose loads are in flight together: 16 x 128-bit loads per lane whatever the width of a row
  // (K = 1000, w = 15: four rows, 250 registers, 8 warps per SM 94.5 us; two rows, 168 registers, 12 warps 83.7 us)
  constexpr int RB = (NT >= 6) ? 2 : 4;
  const int nbatch = (d.W + RB - 1) / RB;
  int qc[NT];
  bool live[NT];  // does this lane own real columns in group t?
#pragma unroll
  for (int t = 0; t < NT; ++t) {
    live[t] = lane + 32 * t < Kq;
    qc[t] = min(lane + 32 * t, Kq - 1);
  }

  // tickets: the first npairs tickets are worth two windows each, later ones a single window, so that the
  // warps run out of work at nearly the same time (share of the ticketed windows that go out in pairs,
  // forward pass inside the step loop / back to back at K=400, batch 10000: 100 % 24.6 / 25.6 us,
  // 60 % 23.8 / 23.5, 30 % 23.8 / 23.0, 0 % 23.9 / 22.6)
  constexpr int FWD_PAIR_PCT = 60;
  constexpr int SINGLE = 1 << 30;
  const int npairs = (int)(((long long)max(d.B - nwarps, 0) * FWD_PAIR_PCT / 100) >> 1);
  int jlast = j;  // last window of the block this warp currently owns
  while (j < d.B) {
    // decide on the next window now; its ids are fetched while this one is summed.  Most windows
    // beyond the first round are handed out in pairs: same-address atomics complete at about
    // one per nanosecond, so one ticket per window all the way would load that one address.
    int jn = j + 1;
    const bool need_ticket = (j >= jlast);
    if (need_ticket && lane == 0) {
      const int t = (int)atomicAdd(&d.ctl->fwd_next[par], 1u);
      jn = (t < npairs) ? nwarps + 2 * t : (nwarps + npairs + t) | SINGLE;
    }
    int winner = -1;
    float awv = 0.f;
    int n_my = -1;
    // hot-row number of this lane's input row; used once the winner is known
    const int hrow = (d.nhot && my >= 0) ? (int)__ldg(d.hotidx + my) : -1;
    if (__shfl_sync(FULL, my, 0) != -2) {  // -2 marks a window past the end of the order
      const int row_id = (my < 0) ? zrow : my;  // lanes >= W hold -1
      unsigned long long acc[NT][2];
#pragma unroll
      for (int t = 0; t < NT; ++t) acc[t][0] = acc[t][1] = 0ull;
      for (int b = 0; b < nbatch; ++b) {
        const ulonglong2* __restrict__ r[RB];
#pragma unroll
        for (int u = 0; u < RB; ++u) {
          const int id = __shfl_sync(FULL, row_id, (RB * b + u) & 31);
          r[u] = reinterpret_cast<const ulonglong2*>(d.wt + (size_t)id * d.Kp);
        }
        ulonglong2 v[RB][NT];
#pragma unroll
        for (int u = 0; u < RB; ++u)
#pragma unroll
          for (int t = 0; t < NT; ++t) v[u][t] = __ldg(r[u] + qc[t]);
        if (b == 0) {
          jn = __shfl_sync(FULL, jn, 0);
          if (need_ticket) {
            jlast = (jn & SINGLE) ? (jn & ~SINGLE) : jn + 1;
            jn &= ~SINGLE;
          }
          if (jn < d.B && lane < d.W) n_my = idx_own[(size_t)jn * d.W + lane];
        }
#pragma unroll
        for (int u = 0; u < RB; ++u)  // position order, as the reference adds
#pragma unroll
          for (int t = 0; t < NT; ++t) {
            add2(acc[t][0], v[u][t].x);
            add2(acc[t][1], v[u][t].y);
          }
      }
      // scaled activations; padding columns and clamped lanes are pushed to -inf
      float a[NT][4];
      float lmax = -INFINITY;
#pragma unroll
      for (int t = 0; t < NT; ++t) {
        const float4 al = *reinterpret_cast<const float4*>(s_alpha + 4 * qc[t]);
        a[t][0] = lo_f(acc[t][0]) * al.x;
        a[t][1] = hi_f(acc[t][0]) * al.y;
        a[t][2] = lo_f(acc[t][1]) * al.z;
        a[t][3] = hi_f(acc[t][1]) * al.w;
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          if (!live[t] || 4 * qc[t] + k >= d.K) a[t][k] = -INFINITY;
          lmax = fmaxf(lmax, a[t][k]);
        }
      }
      const float M = warp_max(lmax);
      const float thr = M - theta;
      int near = 0, cand = 0;
#pragma unroll
      for (int t = 0; t < NT; ++t)
#pragma unroll
        for (int k = 0; k < 4; ++k)
          if (a[t][k] >= thr) {
            ++near;
            cand = 4 * qc[t] + k;
          }
      const int total = __reduce_add_sync(FULL, near);
      if (total == 1 && !force64) {
        const unsigned holder = __ballot_sync(FULL, near != 0);
        winner = __shfl_sync(FULL, cand, __ffs(holder) - 1);
      } else {
        winner = exact_winner(d.wt, alpha, d.Kp, Kq, d.K, d.W, zrow, my, lane, -1);
      }
      awv = weighted_activation(d, alpha, my, winner, lane);
      if (d.has_delta) {
        // the m-th (second) largest raw activation (cuda_funcs.cu:488-561 with m = 2): same certificate
        // with the winner taken out; the reference masks the winner with -9999.9999, which only differs
        // from leaving it out when every other activation lies below that value
        float lmax2 = -INFINITY;
#pragma unroll
        for (int t = 0; t < NT; ++t)
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            if (4 * qc[t] + k == winner) a[t][k] = -INFINITY;
            lmax2 = fmaxf(lmax2, a[t][k]);
          }
        const float M2 = warp_max(lmax2);
        const float thr2 = M2 - theta;
        int near2 = 0, cand2 = 0;
#pragma unroll
        for (int t = 0; t < NT; ++t)
#pragma unroll
          for (int k = 0; k < 4; ++k)
            if (a[t][k] >= thr2) {
              ++near2;
              cand2 = 4 * qc[t] + k;
            }
        const int total2 = __reduce_add_sync(FULL, near2);
        int second;
        if (total2 == 1 && !force64) {
          const unsigned holder = __ballot_sync(FULL, near2 != 0);
          second = __shfl_sync(FULL, cand2, __ffs(holder) - 1);
        } else {
          second = exact_winner(d.wt, alpha, d.Kp, Kq, d.K, d.W, zrow, my, lane, winner);
        }
        const float aw2 = weighted_activation(d, alpha, my, second, lane);
        if (win_out) win_out[d.MO + j] = pk_word((uint32_t)second, seq);
        if (hrow >= 0 && second >= 0) atomicAdd(d.hot_cntn + (size_t)hrow * d.Kp + second, 1u);
        if (lane == 0 && second >= 0) xx_add(second, -d.ctl->delta * aw2, j);  // cuda_funcs.cu:726-735
      }
    } else {
      jn = __shfl_sync(FULL, jn, 0);
      if (need_ticket) {
        jlast = (jn & SINGLE) ? (jn & ~SINGLE) : jn + 1;
        jn &= ~SINGLE;
      }
      if (jn < d.B && lane < d.W) n_my = idx_own[(size_t)jn * d.W + lane];
    }
    if (win_out) {
      win_out[j] = pk_word((uint32_t)winner, seq);
      if (d.has_delta && winner < 0) win_out[d.MO + j] = pk_word((uint32_t)-1, seq);
    }
    if (lane == 0 && winner >= 0) xx_add(winner, awv, j);
    if (hrow >= 0 && winner >= 0) atomicAdd(d.hot_cnt + (size_t)hrow * d.Kp + winner, 1u);
    j = jn;
    my = n_my;
  }
}

// ---------------------------------------------------------------------------
// xx of this rank: one CTA turns the fixed-point sums k_forward left behind into floats, clears
// the accumulators for the next step and puts xx behind the winners in this rank's packet -- and,
// with peer mailboxes, straight into every peer's copy of it.
//
// A unit that won windows but whose activations add up to exactly zero counts as inactive on
// this rank (cu_special_reduction.cu:42-66 tests xx != 0), yet its windows exist; it is published
// as -0.0f so that consumers, which tag every window without knowing xx, can take this rank's
// windows out again (k_scan).  Units that won nothing are +0.0f.
// ---------------------------------------------------------------------------
constexpr uint32_t XX_WON_ZERO = 0x80000000u;
constexpr int XX_THREADS = 512;
constexpr int XX_WARPS = XX_THREADS / 32;
// shared-memory hash table of the tagging kernel: 2 * UN * XX_THREADS slots, at most half full
constexpr size_t tag_table_bytes(int un) { return un > 1 ? (size_t)(2 * 2 * un + 2 * un) * XX_THREADS * sizeof(uint32_t) : 0; }
__device__ __forceinline__ void xx_finish(const Dev& d, int local) {
  const int parity = (int)((d.tick0 + local) & 1);
  const bool mailbox = d.peers != nullptr && d.G > 1;
  const uint32_t seq = (uint32_t)(d.tick0 + local + 1);
  const int kexp = d.ctl->xx_kexp;
  for (int mu = threadIdx.x; mu < d.Kp; mu += XX_THREADS) {
    float x = 0.f;
    if (mu < d.K) {
      const uint32_t wins = __ldcg(d.xx_wins + mu);
      if (wins) {
        unsigned long long h[XX_SLOTS], l[XX_SLOTS];
#pragma unroll
        for (int s = 0; s < XX_SLOTS; ++s) {
          h[s] = __ldcg(d.xx_hi + s * d.Kp + mu);
          l[s] = __ldcg(d.xx_lo + s * d.Kp + mu);
        }
        unsigned long long hi = 0ull, lo = 0ull;  // integer sums: any order gives the same result
#pragma unroll
        for (int s = 0; s < XX_SLOTS; ++s) {
          hi += h[s];
          lo += l[s];
          d.xx_hi[s * d.Kp + mu] = 0ull;
          d.xx_lo[s * d.Kp + mu] = 0ull;
        }
        x = (float)(ldexp((double)(long long)hi, 32 - kexp) + ldexp((double)lo, -kexp));
        if (x == 0.f) x = __uint_as_float(XX_WON_ZERO);
        d.xx_wins[mu] = 0u;
      }
    }
    const unsigned long long word = pk_word(__float_as_uint(x), seq);
    if (mailbox) {
      for (int r = 0; r < d.G; ++r) store_relaxed_sys64(peer_packet(d, r, parity, d.rank) + d.XO + mu, word);
    } else {
      packet(d, parity, d.rank)[d.XO + mu] = word;
    }
  }
  if (threadIdx.x == 0) d.ctl->fwd_next[parity] = 0u;  // rank emulation runs several forward passes per step
}
// The winners of this rank's windows are final when k_forward ends.  Push CTA c of n copies its
// slice of the flagged words into every peer's copy of this rank's packet: plain 8-byte stores over
// NVLink, no fence and no separate flag -- every word announces itself.
constexpr int PUSH_CTAS = 8;
constexpr int HOT_PUSH_CTAS = 0;  // further CTAs that would send the hot-pair counts beside the winners: measured no gain on two GPUs,
                                  // and every CTA taken from the tagging pushes large steps towards more slots per thread
__device__ __forceinline__ void push_winners(const Dev& d, int parity, int cta, int nctas) {
  const ulonglong2* __restrict__ src2 = reinterpret_cast<const ulonglong2*>(packet(d, parity, d.rank));
  const int n2 = d.XO >> 1;  // first and (with delta) second winners, two words at a time
  const int per = (n2 + nctas - 1) / nctas;
  const int hi = min((cta + 1) * per, n2);
  constexpr int PUSH_UNROLL = 4;  // loads of a thread in flight together
  for (int i0 = cta * per + threadIdx.x; i0 < hi; i0 += PUSH_UNROLL * XX_THREADS) {
    ulonglong2 v[PUSH_UNROLL];
#pragma unroll
    for (int u = 0; u < PUSH_UNROLL; ++u)
      if (i0 + u * XX_THREADS < hi) v[u] = __ldcg(src2 + i0 + u * XX_THREADS);
    for (int r = 0; r < d.G; ++r) {
      if (r == d.rank) continue;
      ulonglong2* dst2 = reinterpret_cast<ulonglong2*>(peer_packet(d, r, parity, d.rank));
#pragma unroll
      for (int u = 0; u < PUSH_UNROLL; ++u)
        if (i0 + u * XX_THREADS < hi) dst2[i0 + u * XX_THREADS] = v[u];
    }
  }
}
// The same CTAs then send what this rank's forward pass counted for the hot pairs: every count (zero or not)
// as a flagged word into every rank's hotbox, this rank's own included, and the counters start the next
// step at zero.
__device__ __forceinline__ void push_hot(const Dev& d, int parity, uint32_t seq, int cta, int nctas) {
  const int n = d.nhot * d.Kp;  // pairs per kind
  const int n2 = d.HC >> 1;     // two words at a time
  const int per = (n2 + nctas - 1) / nctas;
  const int hi = min((cta + 1) * per, n2);
  for (int i = cta * per + threadIdx.x; i < hi; i += XX_THREADS) {
    const int v = 2 * i;  // n is even (Kp is a multiple of 4), so a pair of words never straddles the kinds
    uint32_t* src = (v < n) ? d.hot_cnt + v : d.hot_cntn + (v - n);
    const uint2 c = *reinterpret_cast<const uint2*>(src);
    if (c.x | c.y) *reinterpret_cast<uint2*>(src) = make_uint2(0u, 0u);
    const ulonglong2 w = make_ulonglong2(pk_word(c.x, seq), pk_word(c.y, seq));
    for (int r = 0; r < d.G; ++r)
      *reinterpret_cast<ulonglong2*>(hotbox(d, r == d.rank ? d.mail : d.peers[r], parity, d.rank) + v) = w;
  }
}
// Push CTA `cta` of `nctas`: the first PUSH_CTAS send the winners, the others (launched when the hot-pair
// counts travel) the counts, side by side.
__device__ __forceinline__ void serve_exchange(const Dev& d, int parity, uint32_t seq, int cta, int nctas) {
  if (!d.hot_x || nctas <= PUSH_CTAS) {
    push_winners(d, parity, cta, nctas);
    if (d.hot_x) push_hot(d, parity, seq, cta, nctas);
  } else if (cta < PUSH_CTAS) {
    push_winners(d, parity, cta, PUSH_CTAS);
  } else {
    push_hot(d, parity, seq, cta - PUSH_CTAS, nctas - PUSH_CTAS);
  }
}
// CTA 0 finishes xx; further CTAs (when launched) push this rank's winners to the peers.  The tagging
// kernel does both in its first CTAs; this kernel does them alone where xx must be complete before an
// all-gather, and where several ranks share one stream, so that every rank's words are out before any
// rank's tagging looks for them.
__global__ void __launch_bounds__(XX_THREADS) k_xx(Dev d, int local) {
  grid_dependency_wait();
  if (blockIdx.x == 0 && threadIdx.x == 0) phase_mark(d.ctl, PH_XX);
  if (d.ctl->error & FV_DEVERR_TIMEOUT) return;  // a peer never answered: the step loop is void
  if (blockIdx.x == 0) {
    xx_finish(d, local);
  } else {
    serve_exchange(d, (int)((d.tick0 + local) & 1), (uint32_t)(d.tick0 + local + 1), blockIdx.x - 1, gridDim.x - 1);
  }
}

// ---------------------------------------------------------------------------
// T10 bookkeeping.  Every (window, position) of every rank wants to add f_i to the
// matrix position (i, winner).  Each distinct position gets one record
// {position, parked weight, f_i} in a compact list and a count of how many wanted
// it: the claimant parks the weight in the record and leaves TAG_BASE|(record+1) --
// a NaN bit pattern no weight can have -- in its place; later comers for the same
// position find the tag and add to the claimant's count.  A (window, position) is
// skipped when its rank's xx[winner] is zero: the reference drops a replica's whole
// row from the combine in that case (cu_special_reduction.cu:42-66).
// ---------------------------------------------------------------------------
// The first xx_ctas CTAs (one) do not tag: they finish xx (xx_finish) side by side with the tagging;
// with peer mailboxes the next push_ctas CTAs send this rank's winners to the peers.  Tagging needs
// the winners of all ranks (a peer's arrive word by word once its forward pass has ended) but not xx, so it tags every (window, position); a unit that turns out inactive on all
// ranks gets its parked weights back unchanged in k_apply, and the windows of a rank on which the
// unit's xx cancelled to exactly zero are taken out of the counts again by k_scan.
__device__ __forceinline__ void claim_position(const Dev& d, uint32_t pos, uint32_t c, uint32_t slot, uint32_t mult, uint32_t EV) {
  uint32_t* addr = reinterpret_cast<uint32_t*>(d.wt) + pos;
  const uint32_t tag = TAG_BASE | (slot + 1u);
  for (;;) {
    if ((c & ABS_MASK) > TAG_BASE) {
      const uint32_t owner = (c & 0x007fffffu) - 1u;
      if ((c >> 31) || owner >= EV) {
        atomicOr(&d.ctl->error, FV_DEVERR_NAN_WEIGHT);
      } else {
        if (mult & 0xffffu) atomicAdd(&d.cnt[owner], (int)(mult & 0xffffu));
        if (mult >> 16) atomicAdd(&d.cntn[owner], (int)(mult >> 16));
      }
      return;
    }
    const uint32_t prev = atomicCAS(addr, c, tag);
    if (prev == c) {
      // the claimant's own multiplicities travel in the record (first-winner kind in the low half,
      // second-winner kind above); cnt[] only collects later comers, so a position touched from one
      // block costs no counter atomic at all
      const int irow = (int)fdiv(pos, d.mKp, d.sKp);
      d.rec[slot] = make_uint4(pos, c, __float_as_uint(__ldg(d.f + (irow >= d.V ? irow - d.V : irow))), mult);
      return;
    }
    c = prev;
  }
}
// Hot pair v = (hot row, unit): takes what k_forward counted for it (and clears the counters for the next step)
// and claims the position once.  The claimant's record says "one request of each kind present"; the rest of the
// count goes into the counters that later comers use, so that no multiplicity field can overflow.
// What the forward passes counted for hot pair v: this trainer's own counters (cleared here), or, with the
// exchange, the sum of every rank's flagged word (bounded wait for a word that is still on its way).
__device__ __forceinline__ void hot_pair_counts(const Dev& d, int parity, uint32_t seq, int v, uint32_t* c1, uint32_t* c2) {
  if (!d.hot_x) {
    *c1 = __ldcg(d.hot_cnt + v);
    *c2 = d.has_delta ? __ldcg(d.hot_cntn + v) : 0u;
    if (*c1) d.hot_cnt[v] = 0u;
    if (*c2) d.hot_cntn[v] = 0u;
    return;
  }
  const int n = d.nhot * d.Kp;
  uint32_t a = 0u, b = 0u;
  constexpr int RB = 8;  // ranks whose words are fetched together
  for (int r0 = 0; r0 < d.G; r0 += RB) {
    unsigned long long w1[RB], w2[RB];
#pragma unroll
    for (int u = 0; u < RB; ++u) {
      if (r0 + u >= d.G) continue;
      const unsigned long long* box = hotbox(d, d.mail, parity, r0 + u);
      w1[u] = load_relaxed_sys64(box + v);
      w2[u] = d.has_delta ? load_relaxed_sys64(box + n + v) : 0ull;
    }
#pragma unroll
    for (int u = 0; u < RB; ++u) {
      if (r0 + u >= d.G) continue;
      const unsigned long long* box = hotbox(d, d.mail, parity, r0 + u);
      a += ((uint32_t)(w1[u] >> 32) == seq) ? (uint32_t)w1[u] : pk_read(d, box + v, seq, 0u);
      if (d.has_delta) b += ((uint32_t)(w2[u] >> 32) == seq) ? (uint32_t)w2[u] : pk_read(d, box + n + v, seq, 0u);
    }
  }
  *c1 = a;
  *c2 = b;
}
__device__ __forceinline__ void claim_hot_pair(const Dev& d, int v, uint32_t slot, uint32_t EVX, uint32_t c1, uint32_t c2) {
  if (!(c1 | c2)) return;
  const int h = (int)fdiv((uint32_t)v, d.mKp, d.sKp);
  const int mu = v - h * d.Kp;
  const uint32_t pos = (uint32_t)((size_t)__ldg(d.hot_rows + h) * d.Kp + mu);
  uint32_t* addr = reinterpret_cast<uint32_t*>(d.wt) + pos;
  uint32_t c = __ldcg(addr);
  uint32_t owner = slot;
  for (;;) {
    if ((c & ABS_MASK) > TAG_BASE) {
      owner = (c & 0x007fffffu) - 1u;
      if ((c >> 31) || owner >= EVX) {
        atomicOr(&d.ctl->error, FV_DEVERR_NAN_WEIGHT);
        return;
      }
      break;
    }
    const uint32_t prev = atomicCAS(addr, c, TAG_BASE | (slot + 1u));
    if (prev == c) {
      const int irow = __ldg(d.hot_rows + h);
      const uint32_t mult = (c1 ? 1u : 0u) | (c2 ? 0x10000u : 0u);
      d.rec[slot] = make_uint4(pos, c, __float_as_uint(__ldg(d.f + (irow >= d.V ? irow - d.V : irow))), mult);
      c1 -= c1 ? 1u : 0u;
      c2 -= c2 ? 1u : 0u;
      break;
    }
    c = prev;
  }
  if (c1) atomicAdd(&d.cnt[owner], (int)c1);
  if (c2) atomicAdd(&d.cntn[owner], (int)c2);
}
template <int UN>  // slots per thread and block round: a CTA deduplicates UN * XX_THREADS slots together
__global__ void __launch_bounds__(XX_THREADS, 3) k_tag(Dev d, int local, const int32_t* __restrict__ idx, int xx_ctas, int push_ctas) {
  grid_dependency_wait();
  extern __shared__ __align__(16) unsigned char tag_smem[];
  const int parity = (int)((d.tick0 + local) & 1);
  if ((int)blockIdx.x < xx_ctas) {
    xx_finish(d, local);
    return;
  }
  const int svc = xx_ctas + push_ctas;  // CTAs that serve the exchange instead of tagging
  if ((int)blockIdx.x < svc) {
    serve_exchange(d, parity, (uint32_t)(d.tick0 + local + 1), blockIdx.x - xx_ctas, push_ctas);
    return;
  }
  if ((int)blockIdx.x == svc && threadIdx.x == 0) phase_mark(d.ctl, PH_TAG);
  const uint32_t seq = (uint32_t)(d.tick0 + local + 1);
  // Stage 1: a block of TAG_BLOCK slots is deduplicated in a shared-memory hash table keyed by the
  // matrix position, so a (unit, token) pair that occurs many times in the block -- frequent tokens
  // do -- reaches global memory once, with its multiplicity.  Same-address global atomics complete
  // at about one per nanosecond, which made the duplicates of the hottest pairs the bottleneck.
  // Stage 2: the distinct positions are compacted, get record slots (one counter bump per block) and
  // are claimed with one CAS each, the loads of a thread's claims issued together; the winner of a
  // claim writes the record, the others add their multiplicity to the claimant's count.
  __shared__ uint32_t s_scan[XX_WARPS];
  __shared__ uint32_t s_gbase;
  // With delta != 0 every (window, position) contributes twice: +f_i to the first winner's row and
  // -delta*f_i to the second winner's row (cuda_funcs.cu:665-668).  Virtual slot ev = kind * E + e.
  const int E = d.G * d.B * d.W;
  const int EV = E * (1 + d.has_delta);
  constexpr int TAG_BLOCK = UN * XX_THREADS;
  const int nblocks = (EV + (UN == 1 ? d.nhot * d.Kp : 0) + TAG_BLOCK - 1) / TAG_BLOCK;
  const int lane = threadIdx.x & 31, wic = threadIdx.x >> 5;
  const bool emulate = (d.flags & FV_FLAG_EMULATE_RANKS) != 0;
  auto slot_rank = [&](int e) -> int { return (int)fdiv(fdiv((uint32_t)e, d.mW, d.sW), d.mB, d.sB); };
  // packet word with the winner of virtual slot ev (which must be < EV)
  auto winner_word = [&](int ev) -> const unsigned long long* {
    const int kind = (ev >= E) ? 1 : 0;
    const uint32_t q = fdiv((uint32_t)(ev - kind * E), d.mW, d.sW);  // window of the global step
    const uint32_t r = fdiv(q, d.mB, d.sB);                          // its rank
    return packet(d, parity, (int)r) + kind * d.MO + (int)(q - r * (uint32_t)d.B);
  };
  // a peer's winner may still be on its way: the word says so (bounded wait; -1 after a timeout).
  // `first` is the word as a plain load found it, so that several loads can be in flight together.
  auto winner_from = [&](const unsigned long long* word, unsigned long long first) -> int {
    if ((uint32_t)(first >> 32) == seq) return (int)(uint32_t)first;
    return (int)pk_read(d, word, seq, (uint32_t)-1);
  };
  // every rank begins with the blocks of its own windows, whose winners are here already
  const int first_blk = (int)(((long long)nblocks * d.rank) / d.G);
  for (int b0 = blockIdx.x - svc; b0 < nblocks; b0 += gridDim.x - svc) {
    const int blk = (b0 + first_blk) % nblocks;
    if constexpr (UN == 1) {
      // small steps: duplicates inside 512 slots are rare, so skip the table: number the live slots of
      // the CTA with a ballot/prefix (one counter bump per CTA round) and claim directly
      // the winner's address does not depend on the id: both loads leave together
      const int ev = blk * TAG_BLOCK + threadIdx.x;
      // behind the slots, one thread per hot pair: what k_forward counted for it is claimed once, with the count
      if (ev >= EV && ev < EV + d.nhot * d.Kp) {
        uint32_t c1, c2;
        hot_pair_counts(d, parity, seq, ev - EV, &c1, &c2);
        claim_hot_pair(d, ev - EV, (uint32_t)ev, (uint32_t)(EV + d.nhot * d.Kp), c1, c2);
      }
      const int i0 = (ev < EV) ? step_id(d, idx, ev >= E ? ev - E : ev) : -1;
      const unsigned long long* ww = winner_word(ev < EV ? ev : 0);
      const unsigned long long w0 = load_relaxed_sys64(ww);
      const int mu0 = (ev < EV) ? winner_from(ww, w0) : -1;
      bool go0 = i0 >= 0 && mu0 >= 0 &&
                 !(d.shard && (int)((uint32_t)i0 - fdiv((uint32_t)i0, d.mG, d.sG) * (uint32_t)d.G) != d.rank);
      // a hot row's slot of a window k_forward ran here is in the pair's count already
      if (go0 && d.nhot && __ldg(d.hotidx + i0) >= 0 && (emulate || d.hot_x || slot_rank(ev >= E ? ev - E : ev) == d.rank)) go0 = false;
      const uint32_t pos = (uint32_t)((size_t)(go0 ? i0 : 0) * d.Kp + (go0 ? mu0 : 0));
      uint32_t c0 = 0u;
      if (go0) c0 = __ldcg(reinterpret_cast<const uint32_t*>(d.wt) + pos);
      if (!d.shard) {
        // The record of a slot is the slot itself: no numbering, hence no counter to bump and no block barrier
        // in this kernel's chain of dependent accesses.  Slots that own no position stay holes, of which the
        // later kernels skip a few more than a compact list would hold (duplicates inside one step of one
        // rank are rare).  The list is then as long as the step has slots.
        if (blk == 0 && threadIdx.x == 0) d.ctl->list_count[parity] = (uint32_t)(EV + d.nhot * d.Kp);
        if (go0) claim_position(d, pos, c0, (uint32_t)ev, ev >= E ? 0x10000u : 1u, (uint32_t)(EV + d.nhot * d.Kp));
      } else {
        // sharded update: the list is sent to the peers, so it is kept compact
        const unsigned live = __ballot_sync(FULL, go0);
        if (lane == 0) s_scan[wic] = (uint32_t)__popc(live);
        __syncthreads();
        uint32_t before = 0u, tot = 0u;
#pragma unroll
        for (int w = 0; w < XX_WARPS; ++w) {
          const uint32_t c = s_scan[w];
          before += (w < wic) ? c : 0u;
          tot += c;
        }
        if (threadIdx.x == 0) s_gbase = tot ? atomicAdd(&d.ctl->list_count[parity], tot) : 0u;
        __syncthreads();
        if (go0) claim_position(d, pos, c0, s_gbase + before + (uint32_t)__popc(live & ((1u << lane) - 1u)), ev >= E ? 0x10000u : 1u, (uint32_t)EV);
      }
    } else {
      constexpr int TAG_TABLE = 2 * TAG_BLOCK;
      constexpr int TAG_TABLE_LOG2 = (UN == 2) ? 11 : 12;
      static_assert(UN == 2 || UN == 4, "table sizes are worked out for 1024 and 2048 slots per block");
      static_assert((1 << TAG_TABLE_LOG2) == TAG_TABLE, "table size");
      uint32_t* s_key = reinterpret_cast<uint32_t*>(tag_smem);           // [TAG_TABLE] position + 1, 0 = free
      uint32_t* s_cnt = s_key + TAG_TABLE;                               // [TAG_TABLE] two 16-bit multiplicities
      uint32_t* s_ckey = s_cnt + TAG_TABLE;                              // [TAG_BLOCK] compacted keys
      uint32_t* s_cmult = s_ckey + TAG_BLOCK;                            // [TAG_BLOCK] and their multiplicities
      constexpr int NQ = TAG_TABLE / XX_THREADS / 4;  // uint4 groups of the table a thread owns
#pragma unroll
      for (int g = 0; g < NQ; ++g) {
        reinterpret_cast<uint4*>(s_key)[threadIdx.x * NQ + g] = make_uint4(0u, 0u, 0u, 0u);
        reinterpret_cast<uint4*>(s_cnt)[threadIdx.x * NQ + g] = make_uint4(0u, 0u, 0u, 0u);
      }
      __syncthreads();
      int i[UN], mu[UN];
#pragma unroll
      for (int u = 0; u < UN; ++u) {
        const int ev = blk * TAG_BLOCK + u * XX_THREADS + threadIdx.x;
        i[u] = (ev < EV) ? step_id(d, idx, ev >= E ? ev - E : ev) : -1;
      }
      const unsigned long long* ww[UN];
      unsigned long long w0[UN];
#pragma unroll
      for (int u = 0; u < UN; ++u) {  // the winner's address does not depend on the id: all loads leave together
        const int ev = blk * TAG_BLOCK + u * XX_THREADS + threadIdx.x;
        ww[u] = winner_word(ev < EV ? ev : 0);
        w0[u] = load_relaxed_sys64(ww[u]);
      }
#pragma unroll
      for (int u = 0; u < UN; ++u) {
        const int ev = blk * TAG_BLOCK + u * XX_THREADS + threadIdx.x;
        mu[u] = (ev < EV) ? winner_from(ww[u], w0[u]) : -1;
      }
#pragma unroll
      for (int u = 0; u < UN; ++u) {
        // sharded: another rank may own this row
        const bool go = i[u] >= 0 && !(d.shard && (int)((uint32_t)i[u] - fdiv((uint32_t)i[u], d.mG, d.sG) * (uint32_t)d.G) != d.rank);
        if (!go) mu[u] = -1;
      }
#pragma unroll
      for (int u = 0; u < UN; ++u) {
        if (mu[u] < 0) continue;
        const int ev = blk * TAG_BLOCK + u * XX_THREADS + threadIdx.x;
        const uint32_t key = (uint32_t)((size_t)i[u] * d.Kp + mu[u]) + 1u;
        uint32_t h = (key * 2654435761u) >> (32 - TAG_TABLE_LOG2);
        for (;;) {
          const uint32_t old = atomicCAS(&s_key[h], 0u, key);
          if (old == 0u || old == key) {
            atomicAdd(&s_cnt[h], ev >= E ? 0x10000u : 1u);  // a block has <= 2048 slots: 16 bits each suffice
            break;
          }
          h = (h + 1) & (TAG_TABLE - 1);
        }
      }
      __syncthreads();
      // compaction: every thread owns 4 * NQ consecutive table slots
      uint4 k4[NQ], c4[NQ];
      int occ = 0;
#pragma unroll
      for (int g = 0; g < NQ; ++g) {
        k4[g] = reinterpret_cast<const uint4*>(s_key)[threadIdx.x * NQ + g];
        c4[g] = reinterpret_cast<const uint4*>(s_cnt)[threadIdx.x * NQ + g];
        occ += (k4[g].x != 0u) + (k4[g].y != 0u) + (k4[g].z != 0u) + (k4[g].w != 0u);
      }
      int incl = occ;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int v = __shfl_up_sync(FULL, incl, o);
        if (lane >= o) incl += v;
      }
      if (lane == 31) s_scan[wic] = (uint32_t)incl;
      __syncthreads();
      uint32_t before = 0u, tot = 0u;
#pragma unroll
      for (int w = 0; w < XX_WARPS; ++w) {
        const uint32_t c = s_scan[w];
        before += (w < wic) ? c : 0u;
        tot += c;
      }
      if (threadIdx.x == 0) s_gbase = tot ? atomicAdd(&d.ctl->list_count[parity], tot) : 0u;
      uint32_t at = before + (uint32_t)(incl - occ);
#pragma unroll
      for (int g = 0; g < NQ; ++g) {
        if (k4[g].x) { s_ckey[at] = k4[g].x; s_cmult[at] = c4[g].x; ++at; }
        if (k4[g].y) { s_ckey[at] = k4[g].y; s_cmult[at] = c4[g].y; ++at; }
        if (k4[g].z) { s_ckey[at] = k4[g].z; s_cmult[at] = c4[g].z; ++at; }
        if (k4[g].w) { s_ckey[at] = k4[g].w; s_cmult[at] = c4[g].w; ++at; }
      }
      __syncthreads();
      // claims: at most TAG_BLOCK = UN * XX_THREADS compacted positions, UN per thread, loads together
      uint32_t key[UN], cur[UN];
#pragma unroll
      for (int u = 0; u < UN; ++u) {
        const uint32_t cidx = (uint32_t)(u * XX_THREADS + threadIdx.x);
        key[u] = (cidx < tot) ? s_ckey[cidx] : 0u;
        cur[u] = key[u] ? __ldcg(reinterpret_cast<const uint32_t*>(d.wt) + (key[u] - 1u)) : 0u;
      }
      // the claims of a thread leave together: a claim is one compare-and-swap whose answer is either the
      // expected weight (this record owns the position) or the tag of the record that got there first
      uint32_t prev[UN];
#pragma unroll
      for (int u = 0; u < UN; ++u) {
        const uint32_t cidx = (uint32_t)(u * XX_THREADS + threadIdx.x);
        prev[u] = cur[u];
        if (key[u] && (cur[u] & ABS_MASK) <= TAG_BASE)
          prev[u] = atomicCAS(reinterpret_cast<uint32_t*>(d.wt) + (key[u] - 1u), cur[u], TAG_BASE | (s_gbase + cidx + 1u));
      }
#pragma unroll
      for (int u = 0; u < UN; ++u) {
        if (!key[u]) continue;
        const uint32_t cidx = (uint32_t)(u * XX_THREADS + threadIdx.x);
        const uint32_t pos = key[u] - 1u, mult = s_cmult[cidx];
        if (prev[u] == cur[u] && (cur[u] & ABS_MASK) <= TAG_BASE) {
          const int irow = (int)fdiv(pos, d.mKp, d.sKp);
          d.rec[s_gbase + cidx] = make_uint4(pos, cur[u], __float_as_uint(__ldg(d.f + (irow >= d.V ? irow - d.V : irow))), mult);
        } else {
          const uint32_t owner = (prev[u] & 0x007fffffu) - 1u;
          if ((prev[u] & ABS_MASK) <= TAG_BASE || (prev[u] >> 31) || owner >= (uint32_t)EV) {
            atomicOr(&d.ctl->error, FV_DEVERR_NAN_WEIGHT);  // neither the expected weight nor a tag
          } else {
            if (mult & 0xffffu) atomicAdd(&d.cnt[owner], (int)(mult & 0xffffu));
            if (mult >> 16) atomicAdd(&d.cntn[owner], (int)(mult >> 16));
          }
        }
      }
    }
    if (UN != 1 || d.shard) __syncthreads();  // the tables are reused by the next round
  }
}

// Tagging with U slots per thread, for steps with more slots than resident threads (several ranks).
// Every stage is issued for all U slots of a thread before any result is used -- the ids, the winners,
// the weights, and then the claims themselves: a claim is ONE compare-and-swap whose answer is either
// the weight that was expected (this slot owns the position and writes the record) or the tag of the
// slot that got there first (this slot adds its multiplicity to that record's count); no retry is
// needed, because during this kernel a weight can only turn into a tag.  So a block round costs the
// same chain of dependent accesses as one slot per thread, and one round covers the step.
// OWN: the sharded update -- a rank claims only the positions of the rows it owns (i % G == rank).
template <int U, bool OWN>
__global__ void __launch_bounds__(XX_THREADS, 3) k_tag_batch(Dev d, int local, const int32_t* __restrict__ idx, int xx_ctas, int push_ctas) {
  grid_dependency_wait();
  const int parity = (int)((d.tick0 + local) & 1);
  if ((int)blockIdx.x < xx_ctas) {
    xx_finish(d, local);
    return;
  }
  const int svc = xx_ctas + push_ctas;  // CTAs that serve the exchange instead of tagging
  if ((int)blockIdx.x < svc) {
    serve_exchange(d, parity, (uint32_t)(d.tick0 + local + 1), blockIdx.x - xx_ctas, push_ctas);
    return;
  }
  if ((int)blockIdx.x == svc && threadIdx.x == 0) phase_mark(d.ctl, PH_TAG);
  const uint32_t seq = (uint32_t)(d.tick0 + local + 1);
  __shared__ uint32_t s_scan[XX_WARPS];
  __shared__ uint32_t s_gbase;
  // With delta != 0 every (window, position) contributes twice: +f_i to the first winner's row and
  // -delta*f_i to the second winner's row (cuda_funcs.cu:665-668).  Virtual slot ev = kind * E + e.
  const int E = d.G * d.B * d.W;
  const int EV = E * (1 + d.has_delta);
  constexpr int TAG_BLOCK = U * XX_THREADS;
  const int nblocks = (EV + TAG_BLOCK - 1) / TAG_BLOCK;
  const int lane = threadIdx.x & 31, wic = threadIdx.x >> 5;
  const bool emulate = (d.flags & FV_FLAG_EMULATE_RANKS) != 0;
  uint32_t* __restrict__ wbits = reinterpret_cast<uint32_t*>(d.wt);
  // every rank begins with the blocks of its own windows, whose winners are here already
  const int first_blk = (int)(((long long)nblocks * d.rank) / d.G);
  for (int b0 = blockIdx.x - svc; b0 < nblocks; b0 += gridDim.x - svc) {
    const int blk = (b0 + first_blk) % nblocks;
    int i[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int ev = blk * TAG_BLOCK + u * XX_THREADS + threadIdx.x;
      i[u] = (ev < EV) ? step_id(d, idx, ev >= E ? ev - E : ev) : -1;
    }
    const unsigned long long* ww[U];
    unsigned long long w0[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int ev = blk * TAG_BLOCK + u * XX_THREADS + threadIdx.x;
      bool mine = i[u] >= 0;
      if (OWN) mine = mine && (int)((uint32_t)i[u] - fdiv((uint32_t)i[u], d.mG, d.sG) * (uint32_t)d.G) == d.rank;
      const int kind = (mine && ev >= E) ? 1 : 0;
      const uint32_t q = fdiv((uint32_t)(mine ? ev - kind * E : 0), d.mW, d.sW);  // window of the global step
      const uint32_t r = fdiv(q, d.mB, d.sB);                                    // its rank
      // a hot row's slot of a window k_forward ran here is in the pair's count already
      if (!OWN && mine && d.nhot && __ldg(d.hotidx + i[u]) >= 0 && (emulate || d.hot_x || (int)r == d.rank)) mine = false;
      if (!mine) i[u] = -1;
      ww[u] = packet(d, parity, (int)r) + kind * d.MO + (int)(q - r * (uint32_t)d.B);
      w0[u] = mine ? load_relaxed_sys64(ww[u]) : 0ull;
    }
    uint32_t pos[U], c0[U];
    bool go[U];
    uint32_t mine_n = 0u;
#pragma unroll
    for (int u = 0; u < U; ++u) {
      int mu = -1;
      // a peer's winner may still be on its way: the word says so (bounded wait; -1 after a timeout)
      if (i[u] >= 0) mu = ((uint32_t)(w0[u] >> 32) == seq) ? (int)(uint32_t)w0[u] : (int)pk_read(d, ww[u], seq, (uint32_t)-1);
      go[u] = mu >= 0;
      pos[u] = go[u] ? (uint32_t)((size_t)i[u] * d.Kp + mu) : 0u;
      c0[u] = go[u] ? __ldcg(wbits + pos[u]) : 0u;
      mine_n += go[u] ? 1u : 0u;
    }
    uint32_t incl = mine_n;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const uint32_t v = __shfl_up_sync(FULL, incl, o);
      if (lane >= o) incl += v;
    }
    if (lane == 31) s_scan[wic] = incl;
    __syncthreads();
    uint32_t before = 0u, tot = 0u;
#pragma unroll
    for (int w = 0; w < XX_WARPS; ++w) {
      const uint32_t c = s_scan[w];
      before += (w < wic) ? c : 0u;
      tot += c;
    }
    if (threadIdx.x == 0) s_gbase = tot ? atomicAdd(&d.ctl->list_count[parity], tot) : 0u;
    __syncthreads();
    const uint32_t slot0 = s_gbase + before + incl - mine_n;
    // the claims of all U slots leave together ...
    uint32_t prev[U], slot[U];
    uint32_t nslot = slot0;
#pragma unroll
    for (int u = 0; u < U; ++u) {
      slot[u] = nslot;
      nslot += go[u] ? 1u : 0u;
      prev[u] = c0[u];
      if (go[u] && (c0[u] & ABS_MASK) <= TAG_BASE) prev[u] = atomicCAS(wbits + pos[u], c0[u], TAG_BASE | (slot[u] + 1u));
    }
    // ... and their answers are used afterwards
#pragma unroll
    for (int u = 0; u < U; ++u) {
      if (!go[u]) continue;
      const int ev = blk * TAG_BLOCK + u * XX_THREADS + threadIdx.x;
      const uint32_t mult = ev >= E ? 0x10000u : 1u;
      if (prev[u] == c0[u] && (c0[u] & ABS_MASK) <= TAG_BASE) {
        // this slot owns the position: the weight is parked in its record
        const int irow = (int)fdiv(pos[u], d.mKp, d.sKp);
        d.rec[slot[u]] = make_uint4(pos[u], c0[u], __float_as_uint(__ldg(d.f + (irow >= d.V ? irow - d.V : irow))), mult);
      } else {
        const uint32_t owner = (prev[u] & 0x007fffffu) - 1u;
        if ((prev[u] & ABS_MASK) <= TAG_BASE || (prev[u] >> 31) || owner >= (uint32_t)d.rec_cap) {
          atomicOr(&d.ctl->error, FV_DEVERR_NAN_WEIGHT);  // neither the expected weight nor a tag
        } else {
          if (mult & 0xffffu) atomicAdd(&d.cnt[owner], 1);
          if (mult >> 16) atomicAdd(&d.cntn[owner], 1);
        }
      }
    }
    __syncthreads();  // s_scan and s_gbase are reused by the next round
  }
  if (!OWN && d.nhot) {
    // behind the slots, the hot pairs: one thread per pair claims what k_forward counted for it; the non-empty
    // pairs of a warp take their record numbers together
    const int npairs = d.nhot * d.Kp;
    const int stride = (gridDim.x - svc) * XX_THREADS;
    for (int v0 = (blockIdx.x - svc) * XX_THREADS + threadIdx.x; v0 - lane < npairs; v0 += stride) {
      uint32_t c1 = 0u, c2 = 0u;
      if (v0 < npairs) hot_pair_counts(d, parity, seq, v0, &c1, &c2);
      const bool has = (c1 | c2) != 0u;
      const unsigned live = __ballot_sync(FULL, has);
      if (!live) continue;
      uint32_t base = 0u;
      if (lane == 0) base = atomicAdd(&d.ctl->list_count[parity], (uint32_t)__popc(live));
      base = __shfl_sync(FULL, base, 0);
      if (has) claim_hot_pair(d, v0, base + (uint32_t)__popc(live & ((1u << lane) - 1u)), (uint32_t)d.rec_cap, c1, c2);
    }
  }
}

// Per-unit combine over ranks: n = number of ranks with xx != 0, X = mean of xx
// over those ranks (the closed form of cu_special_reduction.cu:42-67 applied to
// the -xx*W term).
__device__ __forceinline__ void unit_stats(const Dev& d, int parity, uint32_t seq, int mu, double* X, int* n) {
  double sum = 0.0;
  int cnt = 0;
  constexpr int RB = 8;  // ranks whose words are fetched together
  for (int r0 = 0; r0 < d.G; r0 += RB) {
    unsigned long long w[RB];
#pragma unroll
    for (int u = 0; u < RB; ++u)
      if (r0 + u < d.G) w[u] = load_relaxed_sys64(packet(d, parity, r0 + u) + d.XO + mu);
#pragma unroll
    for (int u = 0; u < RB; ++u) {
      if (r0 + u >= d.G) break;
      uint32_t bits = (uint32_t)w[u];
      // a peer's xx may still be on its way: the word says so (bounded wait; 0 after a timeout)
      if ((uint32_t)(w[u] >> 32) != seq) bits = pk_read(d, packet(d, parity, r0 + u) + d.XO + mu, seq, 0u);
      const float x = __uint_as_float(bits);
      if (x != 0.f) {
        sum += (double)x;
        ++cnt;
      }
    }
  }
  *n = cnt;
  *X = cnt ? sum / (double)cnt : 0.0;
}
// Ranks (bit r) on which unit mu won windows although its xx is exactly zero: their windows were
// tagged like all others and have to leave the counts again.
__device__ __forceinline__ uint32_t unit_cancelled(const Dev& d, int parity, int mu) {
  uint32_t bad = 0u;
  for (int r = 0; r < d.G; ++r)
    if ((uint32_t)packet(d, parity, r)[d.XO + mu] == XX_WON_ZERO) bad |= 1u << r;  // read after unit_stats: the word is there
  return bad;
}
// How often the windows of the ranks in `bad` asked for matrix row `irow` of unit mu, as first
// winner (*np) and as second winner (*nn).  A plain search over those ranks' windows: this only
// runs when activations cancel exactly on one rank while another rank is active for the unit.
// (Scalars instead of the parameter block: a call by reference would put the block on the stack.)
__device__ __noinline__ int2 cancelled_multiplicity(const unsigned long long* __restrict__ packet0, int P, int G, int B, int W, int MO,
                                                    int has_delta, const int32_t* __restrict__ idx, int rstride, int irow, int mu,
                                                    uint32_t bad) {
  int a = 0, b = 0;
  for (int r = 0; r < G; ++r) {
    if (!((bad >> r) & 1u)) continue;
    const unsigned long long* __restrict__ win = packet0 + (size_t)r * P;
    for (int j = 0; j < B; ++j) {
      const bool first = (int)(uint32_t)win[j] == mu;
      const bool second = has_delta && (int)(uint32_t)win[MO + j] == mu;
      if (!first && !second) continue;
      const int32_t* __restrict__ ids = idx + (size_t)r * rstride + (size_t)j * W;
      for (int t = 0; t < W; ++t)
        if (ids[t] == irow) {
          a += first;
          b += second;
        }
    }
  }
  return make_int2(a, b);
}

// ---------------------------------------------------------------------------
// T11.  nc = max |D| with D = -X*W + S.
//   part 1: owners evaluate D at their (touched) position -> ncb (scalar max);
//   part 2: column maxima of |wt| over the untouched positions (tags read as 0)
//           -> colmax; the dense term's maximum is |X*alpha| * colmax.
// Non-negative floats order like their bit patterns, so maxima are integer.
//
// Every thread does both parts: it first loads the count of its slot(s), then
// streams its rows -- a CTA is `groups` lanes of Kq threads, thread (g, q) owns the
// four columns of float4 group q and walks rows g, g + stride, ... eight at a time,
// so every load instruction of a lane covers one whole contiguous row -- and only
// then finishes the slot's dependent loads, whose latency the row stream has hidden.
// ---------------------------------------------------------------------------
constexpr int SCAN_THREADS = 512;
constexpr int SCAN_UNROLL = 8;
__global__ void __launch_bounds__(SCAN_THREADS, 2) k_scan(Dev d, int local, const int32_t* __restrict__ idx) {
  grid_dependency_wait();
  if (blockIdx.x == 0 && threadIdx.x == 0) phase_mark(d.ctl, PH_SCAN);
  if (d.ctl->error & FV_DEVERR_TIMEOUT) return;  // a peer never answered: the step loop is void
  extern __shared__ __align__(16) unsigned char smem_raw[];
  double* sC = reinterpret_cast<double*>(smem_raw);        // X*alpha
  int* sN = reinterpret_cast<int*>(sC + d.Kp);             // active ranks
  uint32_t* sMax = reinterpret_cast<uint32_t*>(sN + d.Kp); // CTA column maxima
  uint32_t* sBad = sMax + d.Kp;                            // ranks whose windows must leave the counts (unit_cancelled)
  const int p = (int)((d.tick0 + local) & 1);
  const int lane = threadIdx.x & 31;
  const double* __restrict__ alpha = d.alpha + p * d.Kp;
  __shared__ int s_any_bad;
  if (threadIdx.x == 0) s_any_bad = 0;
  __syncthreads();
  const uint32_t seq = (uint32_t)(d.tick0 + local + 1);
  for (int mu = threadIdx.x; mu < d.Kp; mu += blockDim.x) {
    double X = 0.0;
    int n = 0;
    if (mu < d.K) unit_stats(d, p, seq, mu, &X, &n);  // waits (bounded) for a peer's xx still on its way
    sC[mu] = X * alpha[mu];
    sN[mu] = n;
    sMax[mu] = 0u;
    if (blockIdx.x == 0) {  // the apply kernel takes the combine from here instead of polling G words per unit again
      d.stat_x[p * d.Kp + mu] = X;
      d.stat_n[p * d.Kp + mu] = n;
    }
    const uint32_t bad = (mu < d.K && n > 0) ? unit_cancelled(d, p, mu) : 0u;
    sBad[mu] = bad;
    if (bad) s_any_bad = 1;
  }
  __syncthreads();
  const int nrec = (int)min(d.ctl->list_count[p], (uint32_t)d.rec_cap);
  const int nthreads = gridDim.x * blockDim.x;
  const int e0 = blockIdx.x * blockDim.x + threadIdx.x;
  if (s_any_bad) {
    // some rank's windows for a unit do not count although the unit is active elsewhere: take them
    // out of this thread's records before anybody (here or in k_apply) reads the counts
    const unsigned long long* packet0 = packet(d, p, 0);
    for (int k = e0; k < nrec; k += nthreads) {
      const uint4 r = d.rec[k];
      if (r.w == 0u) continue;
      const int irow = (int)fdiv(r.x, d.mKp, d.sKp);
      const int mu = (int)r.x - irow * d.Kp;
      if (!sBad[mu]) continue;
      const int2 c = cancelled_multiplicity(packet0, d.P, d.G, d.B, d.W, d.MO, d.has_delta, idx, d.idx_rstride, irow, mu, sBad[mu]);
      if (c.x) d.cnt[k] -= c.x;
      if (c.y) d.cntn[k] -= c.y;
    }
  }

  // part 1, first half: counts and records of this thread's share of the touched-position list
  // (coalesced loads, issued before the row stream so that their latency hides behind it)
  const float delta = d.ctl->delta;
  constexpr int TS = 4;
  float cs[TS];  // net multiplicity of the scatter term: (+1 kind) - delta * (-delta kind)
  uint4 rc[TS];
#pragma unroll
  for (int u = 0; u < TS; ++u) {
    const int k = e0 + u * nthreads;
    const int cp = (k < nrec) ? d.cnt[k] : 0;
    const int cn = (k < nrec && d.has_delta) ? d.cntn[k] : 0;
    rc[u] = (k < nrec) ? d.rec[k] : make_uint4(0u, 0u, 0u, 0u);
    cs[u] = (float)(cp + (int)(rc[u].w & 0xffffu)) - delta * (float)(cn + (int)(rc[u].w >> 16));
    // sharded: the peers learn this record's count now, long before they need it
    if (d.shard && k < nrec) push_entry(d, k, rc[u].w ? (rc[u].x | ENTRY_VALID) : ENTRY_HOLE, cp + (int)(rc[u].w & 0xffffu));
  }

  // part 2: column maxima of |wt| with tags read as 0
  const int Kq = d.Kq;
  const int groups = SCAN_THREADS / Kq;  // Kq <= 256, so at least 2
  const int g = threadIdx.x / Kq, q = threadIdx.x - g * Kq;
  if (g < groups) {
    const int stride = gridDim.x * groups;
    uint32_t m0 = 0u, m1 = 0u, m2 = 0u, m3 = 0u;
    auto fold_in = [&](const uint4& v) {
      uint32_t u;
      u = v.x & ABS_MASK; m0 = max(m0, u > TAG_BASE ? 0u : u);
      u = v.y & ABS_MASK; m1 = max(m1, u > TAG_BASE ? 0u : u);
      u = v.z & ABS_MASK; m2 = max(m2, u > TAG_BASE ? 0u : u);
      u = v.w & ABS_MASK; m3 = max(m3, u > TAG_BASE ? 0u : u);
    };
    const uint4* __restrict__ base = reinterpret_cast<const uint4*>(d.wt) + q;
    // sharded: only the rows this rank owns (rank, rank + G, ...), i.e. row = rank + G * k
    const int rmul = d.shard ? d.G : 1, radd = d.shard ? d.rank : 0;
    const int nrows = d.shard ? (d.N - d.rank + d.G - 1) / d.G : d.N;
    int row = blockIdx.x * groups + g;
    for (; row + (SCAN_UNROLL - 1) * stride < nrows; row += SCAN_UNROLL * stride) {
      uint4 v[SCAN_UNROLL];
#pragma unroll
      for (int u = 0; u < SCAN_UNROLL; ++u) v[u] = __ldcg(base + (size_t)(radd + rmul * (row + u * stride)) * Kq);
#pragma unroll
      for (int u = 0; u < SCAN_UNROLL; ++u) fold_in(v[u]);
    }
    if (row < nrows) {  // ragged end: same unrolled batch, rows past the end re-read the first one
      uint4 v[SCAN_UNROLL];
#pragma unroll
      for (int u = 0; u < SCAN_UNROLL; ++u) {
        const int rr = row + u * stride;
        v[u] = __ldcg(base + (size_t)(radd + rmul * (rr < nrows ? rr : row)) * Kq);
      }
#pragma unroll
      for (int u = 0; u < SCAN_UNROLL; ++u) fold_in(v[u]);
    }
    if (m0) atomicMax(&sMax[4 * q + 0], m0);
    if (m1) atomicMax(&sMax[4 * q + 1], m1);
    if (m2) atomicMax(&sMax[4 * q + 2], m2);
    if (m3) atomicMax(&sMax[4 * q + 3], m3);
  }

  // part 1, second half: exact D at the touched positions (records with a count; reserved
  // records whose position somebody else had claimed keep count 0)
  uint32_t tmax = 0u;
  auto touched = [&](float c, const uint4& r) {
    if (r.w == 0u) return;  // a reserved record nobody claimed
    const int mu = (int)(r.x - fdiv(r.x, d.mKp, d.sKp) * (uint32_t)d.Kp);
    if (sN[mu] == 0) return;  // the unit proved inactive on every rank: no update there
    const double D = -sC[mu] * (double)__uint_as_float(r.y) + (double)c * (double)__uint_as_float(r.z) / (double)sN[mu];
    tmax = max(tmax, __float_as_uint(fabsf((float)D)));
  };
#pragma unroll
  for (int u = 0; u < TS; ++u) touched(cs[u], rc[u]);
  for (int k = e0 + TS * nthreads; k < nrec; k += nthreads) {
    const uint4 r = d.rec[k];
    const int cn = d.has_delta ? d.cntn[k] : 0;
    const int cp = d.cnt[k];
    touched((float)(cp + (int)(r.w & 0xffffu)) - delta * (float)(cn + (int)(r.w >> 16)), r);
    if (d.shard) push_entry(d, k, r.w ? (r.x | ENTRY_VALID) : ENTRY_HOLE, cp + (int)(r.w & 0xffffu));
  }
  __shared__ uint32_t s_tmax;
  if (threadIdx.x == 0) s_tmax = 0u;
  __syncthreads();
  tmax = warp_max_u32(tmax);
  if (lane == 0 && tmax) atomicMax(&s_tmax, tmax);
  __syncthreads();
  if (threadIdx.x == 0 && s_tmax) atomicMax(&d.ncb[p], s_tmax);  // one global atomic per CTA
  for (int mu = threadIdx.x; mu < d.Kp; mu += blockDim.x) {
    const uint32_t v = sMax[mu];
    if (v && v > __ldcg(&d.colmax[p * d.Kp + mu])) atomicMax(&d.colmax[p * d.Kp + mu], v);
  }
  if (!d.shard) return;

  // Sharded update: the CTA that finishes last turns this rank's maxima into its partial
  // normaliser and pushes it, with a flag, into every rank's mailbox (its own included).
  __shared__ unsigned s_last;
  __shared__ float s_red[SCAN_THREADS / 32];
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) s_last = (atomicAdd(&d.ctl->scan_ticket, 1u) == gridDim.x - 1) ? 1u : 0u;
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  float dense = 0.f;
  for (int mu = threadIdx.x; mu < d.K; mu += blockDim.x)
    if (sN[mu] > 0) dense = fmaxf(dense, (float)(fabs(sC[mu]) * (double)__uint_as_float(__ldcg(&d.colmax[p * d.Kp + mu]))));
  dense = warp_max(dense);
  if (lane == 0) s_red[threadIdx.x >> 5] = dense;
  __syncthreads();
  if (threadIdx.x == 0) {
    float nc = __uint_as_float(__ldcg(&d.ncb[p]));
    for (int w = 0; w < SCAN_THREADS / 32; ++w) nc = fmaxf(nc, s_red[w]);
    s_red[0] = nc;
    d.ctl->scan_ticket = 0u;
  }
  __syncthreads();
  if (threadIdx.x < d.G) {
    // the partial normaliser to everybody (this rank included), the length of the entry list to the peers
    const unsigned long long seq = (unsigned)(d.tick0 + local + 1);
    unsigned long long* words = reinterpret_cast<unsigned long long*>(d.peers[threadIdx.x] + WORD_NC);
    store_relaxed_sys64(words + p * MAX_RANKS + d.rank, (seq << 32) | __float_as_uint(s_red[0]));
    unsigned long long* outw = reinterpret_cast<unsigned long long*>(d.peers[threadIdx.x] + WORD_OUT);
    store_relaxed_sys64(outw + p * MAX_RANKS + d.rank, (seq << 32) | (unsigned)nrec);
  }
}

// ---------------------------------------------------------------------------
// Column maxima without streaming the matrix.
//
// nc needs, per active unit mu, the largest |wt[i][mu]| over the rows i the step did NOT touch.  The
// weights only change at touched positions (and when the scales are folded in), so the few rows that
// can hold that maximum are kept from step to step:
//   cand_rows[mu][..]  candidate rows,   cand_floor[mu]  a bound: every scanned row outside the list
//                                                         has |wt| <= floor (bit patterns compare like floats).
// k_eval reads the candidates' current weights -- a tagged one was touched and is skipped -- and takes
// their maximum m.  If m >= floor no row outside the list can beat it: m IS the maximum over untouched
// rows, exactly.  Otherwise (every strong candidate touched in this step) the CTA that queried the unit
// reads the unit's whole column, which gives the exact maximum and its row, lowers the floor to that
// maximum and lists the row.  k_apply keeps the bound true: a touched weight whose new magnitude
// exceeds its unit's floor is listed (or raises the floor when the list is full).  After a fold or
// new weights the lists are rebuilt in the next step by two passes over the matrix: k_colscan finds
// every unit's maximum, k_collect lists every untouched row above CAND_THETA of it.
// With the sharded update a rank keeps lists for the rows it owns.
// ---------------------------------------------------------------------------
constexpr int CAND_CAP = 64;
constexpr float CAND_THETA = 0.85f;  // a rebuild lists the untouched rows above this fraction of their unit's maximum

// Sharded update: this rank's partial normaliser (its records and the columns of its rows) and the length
// of its entry list go to every rank, each in one flagged word.  Run by one CTA once the maxima are final.
__device__ __forceinline__ void publish_partial(const Dev& d, int local, int p) {
  __shared__ float s_pub[SCAN_THREADS / 32];
  const double* __restrict__ alpha = d.alpha + p * d.Kp;
  float dense = 0.f;
  for (int mu = threadIdx.x; mu < d.K; mu += blockDim.x) {
    const int n = __ldcg(d.stat_n + p * d.Kp + mu);
    if (n > 0)
      dense = fmaxf(dense, (float)(fabs(__ldcg(d.stat_x + p * d.Kp + mu) * alpha[mu]) * (double)__uint_as_float(__ldcg(&d.colmax[p * d.Kp + mu]))));
  }
  dense = warp_max(dense);
  if ((threadIdx.x & 31) == 0) s_pub[threadIdx.x >> 5] = dense;
  __syncthreads();
  if (threadIdx.x == 0) {
    float nc = __uint_as_float(__ldcg(&d.ncb[p]));
    for (int w = 0; w < (int)(blockDim.x >> 5); ++w) nc = fmaxf(nc, s_pub[w]);
    s_pub[0] = nc;
  }
  __syncthreads();
  if (threadIdx.x < d.G) {
    const unsigned long long seq = (unsigned)(d.tick0 + local + 1);
    const unsigned nrec = min(d.ctl->list_count[p], (uint32_t)d.rec_cap);
    unsigned long long* words = reinterpret_cast<unsigned long long*>(d.peers[threadIdx.x] + WORD_NC);
    store_relaxed_sys64(words + p * MAX_RANKS + d.rank, (seq << 32) | __float_as_uint(s_pub[0]));
    unsigned long long* outw = reinterpret_cast<unsigned long long*>(d.peers[threadIdx.x] + WORD_OUT);
    store_relaxed_sys64(outw + p * MAX_RANKS + d.rank, (seq << 32) | nrec);
  }
}

// The first half of k_scan (combine, records, exact D at the touched positions) plus the list query.
// The two jobs are chains of dependent memory accesses, so they run side by side in different CTAs:
// the first `qblocks` CTAs query the lists (one warp per unit), the others walk the records.
__global__ void __launch_bounds__(SCAN_THREADS, 2) k_eval(Dev d, int local, const int32_t* __restrict__ idx, int rebuild, int qblocks) {
  grid_dependency_wait();
  if (blockIdx.x == 0 && threadIdx.x == 0) phase_mark(d.ctl, PH_SCAN);
  if (d.ctl->error & FV_DEVERR_TIMEOUT) return;  // a peer never answered: the step loop is void
  const int p = (int)((d.tick0 + local) & 1);
  const int lane = threadIdx.x & 31;
  const uint32_t seq = (uint32_t)(d.tick0 + local + 1);

  if ((int)blockIdx.x < qblocks) {
    // ---- the candidate lists: one warp per unit, a lane per candidate --------------------------
    constexpr int QW = SCAN_THREADS / 32;
    __shared__ int s_unc[QW];
    const int wic = threadIdx.x >> 5;
    const int mu = blockIdx.x * QW + wic;
    if (lane == 0) s_unc[wic] = 0;
    if (mu < d.K && rebuild) {
      // new weights or a fold: every list starts afresh; k_colscan and k_collect follow in this step
      if (lane == 0) {
        d.cand_unc[mu] = 1u;
        d.cand_n[mu] = 0;
      }
    } else if (mu < d.K) {
      // candidates first: their loads do not depend on anything
      const uint32_t* __restrict__ wbits = reinterpret_cast<const uint32_t*>(d.wt);
      const int n = min(__ldcg(d.cand_n + mu), CAND_CAP);
      const uint32_t floor_bits = __ldcg(d.cand_floor + mu);
      int row[CAND_CAP / 32];
#pragma unroll
      for (int t = 0; t < CAND_CAP / 32; ++t) row[t] = (lane + 32 * t < n) ? __ldcg(d.cand_rows + (size_t)mu * CAND_CAP + lane + 32 * t) : -1;
      // is the unit active on any rank?  (lane r looks at rank r's xx; a word still on its way is waited for)
      uint32_t xbits = 0u;
      if (lane < d.G) {
        const unsigned long long* word = packet(d, p, lane) + d.XO + mu;
        const unsigned long long w = load_relaxed_sys64(word);
        xbits = ((uint32_t)(w >> 32) == seq) ? (uint32_t)w : pk_read(d, word, seq, 0u);
      }
      const bool active = __any_sync(FULL, lane < d.G && __uint_as_float(xbits) != 0.f);
      if (active) {  // otherwise no update for this unit: its maximum is not needed
        uint32_t m = 0u;
#pragma unroll
        for (int t = 0; t < CAND_CAP / 32; ++t) {
          if (row[t] < 0) continue;
          const uint32_t w = __ldcg(wbits + (size_t)row[t] * d.Kp + mu) & ABS_MASK;
          m = max(m, w > TAG_BASE ? 0u : w);  // a tag: touched in this step, its exact D is taken at the record
        }
        m = warp_max_u32(m);
        if (lane == 0) {
          if (m >= floor_bits) d.colmax[p * d.Kp + mu] = m;
          else s_unc[wic] = 1;
        }
      }
    }
    __syncthreads();
    // A unit whose strong candidates were all touched in this step: the whole CTA reads the unit's column
    // (tags as 0), which gives the exact maximum and its row; the floor drops to that maximum -- no
    // untouched row exceeds it, and k_apply checks every touched one against it -- and the row is listed.
    for (int w = 0; w < QW; ++w) {
      if (!s_unc[w]) continue;
      const int cu = blockIdx.x * QW + w;
      const uint32_t* __restrict__ col = reinterpret_cast<const uint32_t*>(d.wt) + cu;
      const int rmul = d.shard ? d.G : 1, radd = d.shard ? d.rank : 0;
      const int nrows = d.shard ? (d.N - d.rank + d.G - 1) / d.G : d.N;
      unsigned long long best = 0ull;  // (bits << 32) | row
      constexpr int RU = 8;
      for (int r0 = threadIdx.x; r0 < nrows; r0 += RU * SCAN_THREADS) {
        uint32_t v[RU];
#pragma unroll
        for (int u = 0; u < RU; ++u) {
          const int r = r0 + u * SCAN_THREADS;
          v[u] = (r < nrows) ? (__ldcg(col + (size_t)(radd + rmul * r) * d.Kp) & ABS_MASK) : 0u;
        }
#pragma unroll
        for (int u = 0; u < RU; ++u) {
          const int r = r0 + u * SCAN_THREADS;
          if (r < nrows && v[u] <= TAG_BASE) best = max(best, ((unsigned long long)v[u] << 32) | (uint32_t)(radd + rmul * r));
        }
      }
#pragma unroll
      for (int o = 16; o >= 1; o >>= 1) best = max(best, __shfl_xor_sync(FULL, best, o));
      __shared__ unsigned long long s_best[QW];
      if (lane == 0) s_best[wic] = best;
      __syncthreads();
      if (threadIdx.x == 0) {
        for (int k = 1; k < QW; ++k) best = max(best, s_best[k]);
        const uint32_t m = (uint32_t)(best >> 32);
        d.colmax[p * d.Kp + cu] = m;
        d.cand_floor[cu] = m;
        if (m) {
          const int row = (int)(uint32_t)best;
          const int n = min(d.cand_n[cu], CAND_CAP);
          bool have = false;
          for (int j = 0; j < n; ++j) have |= (d.cand_rows[(size_t)cu * CAND_CAP + j] == row);
          if (!have) {
            // a full list gives up one of its rows: every listed untouched row is <= m, the new floor, and a
            // listed touched row is checked again when k_apply writes its new weight
            const int slot = (n < CAND_CAP) ? n : (int)((d.tick0 + local + (unsigned)cu) % CAND_CAP);
            d.cand_rows[(size_t)cu * CAND_CAP + slot] = row;
            d.cand_n[cu] = (n < CAND_CAP) ? n + 1 : CAND_CAP;
          } else {
            d.cand_n[cu] = n;
          }
        }
        atomicAdd(&d.ctl->scans_run, 1u);
      }
      __syncthreads();
    }
  } else {
  // ---- the records: exact D at the touched positions -------------------------------------------
  extern __shared__ __align__(16) unsigned char smem_raw[];
  double* sC = reinterpret_cast<double*>(smem_raw);        // X*alpha
  int* sN = reinterpret_cast<int*>(sC + d.Kp);             // active ranks
  uint32_t* sBad = reinterpret_cast<uint32_t*>(sN + d.Kp) + d.Kp;  // same layout as k_scan (its column maxima lie between)
  const double* __restrict__ alpha = d.alpha + p * d.Kp;
  __shared__ int s_any_bad;
  const int nrec = (int)min(d.ctl->list_count[p], (uint32_t)d.rec_cap);
  const int nthreads = (gridDim.x - qblocks) * blockDim.x;
  const int e0 = (blockIdx.x - qblocks) * blockDim.x + threadIdx.x;
  constexpr int TS = 4;
  int cp[TS], cn[TS];
  uint4 rc[TS];
  auto load_batch = [&](int k0) {
#pragma unroll
    for (int u = 0; u < TS; ++u) {
      const int k = k0 + u * nthreads;
      cp[u] = (k < nrec) ? d.cnt[k] : 0;
      cn[u] = (k < nrec && d.has_delta) ? d.cntn[k] : 0;
      rc[u] = (k < nrec) ? d.rec[k] : make_uint4(0u, 0u, 0u, 0u);
    }
  };
  load_batch(e0);  // in flight while the combine below polls the packets
  if (threadIdx.x == 0) s_any_bad = 0;
  __syncthreads();
  for (int mu = threadIdx.x; mu < d.Kp; mu += blockDim.x) {
    double X = 0.0;
    int n = 0;
    if (mu < d.K) unit_stats(d, p, seq, mu, &X, &n);  // waits (bounded) for a peer's xx still on its way
    sC[mu] = X * alpha[mu];
    sN[mu] = n;
    if ((int)blockIdx.x == qblocks) {  // the later kernels take the combine from here
      d.stat_x[p * d.Kp + mu] = X;
      d.stat_n[p * d.Kp + mu] = n;
    }
    const uint32_t bad = (mu < d.K && n > 0) ? unit_cancelled(d, p, mu) : 0u;
    sBad[mu] = bad;
    if (bad) s_any_bad = 1;
  }
  __syncthreads();
  if (s_any_bad) {
    // some rank's windows for a unit do not count although the unit is active elsewhere: take them
    // out of this thread's records before anybody (here or in k_apply) reads the counts
    const unsigned long long* packet0 = packet(d, p, 0);
    for (int k = e0; k < nrec; k += nthreads) {
      const uint4 r = d.rec[k];
      if (r.w == 0u) continue;
      const int irow = (int)fdiv(r.x, d.mKp, d.sKp);
      const int mu = (int)r.x - irow * d.Kp;
      if (!sBad[mu]) continue;
      const int2 c = cancelled_multiplicity(packet0, d.P, d.G, d.B, d.W, d.MO, d.has_delta, idx, d.idx_rstride, irow, mu, sBad[mu]);
      if (c.x) d.cnt[k] -= c.x;
      if (c.y) d.cntn[k] -= c.y;
    }
    load_batch(e0);  // the counts have changed
  }
  const float delta = d.ctl->delta;
  uint32_t tmax = 0u;
  for (int k0 = e0; k0 < nrec; k0 += TS * nthreads) {
    if (k0 != e0) load_batch(k0);
#pragma unroll
    for (int u = 0; u < TS; ++u) {
      const int k = k0 + u * nthreads;
      if (k >= nrec) continue;
      const int own = cp[u] + (int)(rc[u].w & 0xffffu);
      // sharded: the peers learn this record's count now, long before they need it
      if (d.shard) push_entry(d, k, rc[u].w ? (rc[u].x | ENTRY_VALID) : ENTRY_HOLE, own);
      if (rc[u].w == 0u) continue;  // a reserved record nobody claimed
      const int mu = (int)(rc[u].x - fdiv(rc[u].x, d.mKp, d.sKp) * (uint32_t)d.Kp);
      if (sN[mu] == 0) continue;    // the unit proved inactive on every rank: no update there
      const float c = (float)own - delta * (float)(cn[u] + (int)(rc[u].w >> 16));
      const double D = -sC[mu] * (double)__uint_as_float(rc[u].y) + (double)c * (double)__uint_as_float(rc[u].z) / (double)sN[mu];
      tmax = max(tmax, __float_as_uint(fabsf((float)D)));
    }
  }
  __shared__ uint32_t s_tmax;
  if (threadIdx.x == 0) s_tmax = 0u;
  __syncthreads();
  tmax = warp_max_u32(tmax);
  if (lane == 0 && tmax) atomicMax(&s_tmax, tmax);
  __syncthreads();
  if (threadIdx.x == 0 && s_tmax) atomicMax(&d.ncb[p], s_tmax);  // one global atomic per CTA
  }  // records
  if (!d.shard || rebuild) return;  // (a rebuild step publishes from k_colscan, once the maxima exist)
  // Sharded update: the CTA that finishes last publishes this rank's partial normaliser.
  __shared__ unsigned s_last_eval;
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) s_last_eval = (atomicAdd(&d.ctl->scan_ticket, 1u) == gridDim.x - 1) ? 1u : 0u;
  __syncthreads();
  if (!s_last_eval) return;
  __threadfence();
  if (threadIdx.x == 0) d.ctl->scan_ticket = 0u;
  publish_partial(d, local, p);
}

// First pass of a rebuild (launched after k_eval in the step that follows new weights or a fold): column
// maxima of |wt| with tags read as 0 and the row of each maximum; the last CTA starts every unit's list
// with that row and leaves the floor at CAND_THETA of the maximum for k_collect.
__global__ void __launch_bounds__(SCAN_THREADS, 2) k_colscan(Dev d, int local, int rebuild) {
  grid_dependency_wait();
  if (d.ctl->error & FV_DEVERR_TIMEOUT) return;
  const int p = (int)((d.tick0 + local) & 1);
  extern __shared__ __align__(16) unsigned char smem_raw[];
  unsigned long long* sArg = reinterpret_cast<unsigned long long*>(smem_raw);  // [Kp] CTA maxima with their rows
  for (int mu = threadIdx.x; mu < d.Kp; mu += blockDim.x) sArg[mu] = 0ull;
  __syncthreads();
  const int Kq = d.Kq;
  const int groups = SCAN_THREADS / Kq;
  const int g = threadIdx.x / Kq, q = threadIdx.x - g * Kq;
  if (g < groups) {
    const int stride = gridDim.x * groups;
    unsigned long long a0 = 0ull, a1 = 0ull, a2 = 0ull, a3 = 0ull;  // (bits << 32) | row
    auto fold_in = [&](const uint4& v, int row) {
      uint32_t u;
      u = v.x & ABS_MASK; a0 = max(a0, ((unsigned long long)(u > TAG_BASE ? 0u : u) << 32) | (uint32_t)row);
      u = v.y & ABS_MASK; a1 = max(a1, ((unsigned long long)(u > TAG_BASE ? 0u : u) << 32) | (uint32_t)row);
      u = v.z & ABS_MASK; a2 = max(a2, ((unsigned long long)(u > TAG_BASE ? 0u : u) << 32) | (uint32_t)row);
      u = v.w & ABS_MASK; a3 = max(a3, ((unsigned long long)(u > TAG_BASE ? 0u : u) << 32) | (uint32_t)row);
    };
    const uint4* __restrict__ base = reinterpret_cast<const uint4*>(d.wt) + q;
    const int rmul = d.shard ? d.G : 1, radd = d.shard ? d.rank : 0;
    const int nrows = d.shard ? (d.N - d.rank + d.G - 1) / d.G : d.N;
    int row = blockIdx.x * groups + g;
    for (; row + (SCAN_UNROLL - 1) * stride < nrows; row += SCAN_UNROLL * stride) {
      uint4 v[SCAN_UNROLL];
#pragma unroll
      for (int u = 0; u < SCAN_UNROLL; ++u) v[u] = __ldcg(base + (size_t)(radd + rmul * (row + u * stride)) * Kq);
#pragma unroll
      for (int u = 0; u < SCAN_UNROLL; ++u) fold_in(v[u], radd + rmul * (row + u * stride));
    }
    for (; row < nrows; row += stride) fold_in(__ldcg(base + (size_t)(radd + rmul * row) * Kq), radd + rmul * row);
    if (a0 >> 32) atomicMax(&sArg[4 * q + 0], a0);
    if (a1 >> 32) atomicMax(&sArg[4 * q + 1], a1);
    if (a2 >> 32) atomicMax(&sArg[4 * q + 2], a2);
    if (a3 >> 32) atomicMax(&sArg[4 * q + 3], a3);
  }
  __syncthreads();
  for (int mu = threadIdx.x; mu < d.Kp; mu += blockDim.x) {
    const unsigned long long v = sArg[mu];
    if ((v >> 32) && v > __ldcg(&d.colarg[mu])) atomicMax(&d.colarg[mu], v);
  }
  // the CTA that finishes last owns the result
  __shared__ unsigned s_last;
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) s_last = (atomicAdd(&d.ctl->scan_ticket, 1u) == gridDim.x - 1) ? 1u : 0u;
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  for (int mu = threadIdx.x; mu < d.K; mu += blockDim.x) {
    const unsigned long long v = __ldcg(&d.colarg[mu]);
    const uint32_t m = (uint32_t)(v >> 32);
    d.colarg[mu] = 0ull;
    if (!d.cand_unc[mu]) continue;  // certified by its list (k_eval wrote the same maximum)
    d.cand_unc[mu] = 0u;
    d.colmax[p * d.Kp + mu] = m;
    // No untouched row exceeds m, so m is a valid floor (touched rows are checked against it by k_apply).
    // A rebuild starts k_collect's threshold from CAND_THETA * m instead.
    d.cand_floor[mu] = rebuild ? __float_as_uint(CAND_THETA * __uint_as_float(m)) : m;
    if (m) {
      const int row = (int)(uint32_t)v;
      int n = min(d.cand_n[mu], CAND_CAP);
      bool have = false;
      for (int j = 0; j < n; ++j) have |= (d.cand_rows[(size_t)mu * CAND_CAP + j] == row);
      if (!have) {
        // a full list gives up one of its rows: every listed untouched row is <= m, the new floor, and a
        // listed touched row is checked again when k_apply writes its new weight
        const int slot = (n < CAND_CAP) ? n : (int)((d.tick0 + local + (unsigned)mu) % CAND_CAP);
        d.cand_rows[(size_t)mu * CAND_CAP + slot] = row;
        d.cand_n[mu] = (n < CAND_CAP) ? n + 1 : CAND_CAP;
      } else {
        d.cand_n[mu] = n;
      }
    }
  }
  if (threadIdx.x == 0) {
    d.ctl->scan_ticket = 0u;
  }
  __syncthreads();
  if (d.shard) publish_partial(d, local, p);
}

// Rebuild, second pass (after k_colscan left every unit's floor at CAND_THETA of its maximum and listed the
// arg-max row): every untouched row above its unit's floor is listed; when a list is full the floor
// rises to the row that did not fit, so the bound stays true.
__global__ void __launch_bounds__(SCAN_THREADS, 2) k_collect(Dev d) {
  grid_dependency_wait();
  if (d.ctl->error & FV_DEVERR_TIMEOUT) return;
  const int Kq = d.Kq;
  const int groups = SCAN_THREADS / Kq;
  const int g = threadIdx.x / Kq, q = threadIdx.x - g * Kq;
  if (g >= groups) return;
  const int stride = gridDim.x * groups;
  const uint4* __restrict__ base = reinterpret_cast<const uint4*>(d.wt) + q;
  const int rmul = d.shard ? d.G : 1, radd = d.shard ? d.rank : 0;
  const int nrows = d.shard ? (d.N - d.rank + d.G - 1) / d.G : d.N;
  uint32_t fl[4];
#pragma unroll
  for (int c = 0; c < 4; ++c) fl[c] = __ldcg(d.cand_floor + min(4 * q + c, d.Kp - 1));
  auto consider = [&](uint32_t bits, int c, int row) {
    const uint32_t u = bits & ABS_MASK;
    const int mu = 4 * q + c;
    if (u > TAG_BASE || u <= fl[c] || mu >= d.K) return;
    if (u <= (fl[c] = __ldcg(d.cand_floor + mu))) return;  // the floor may have risen meanwhile
    // the only row listed before this pass is the arg-max row, in the first place; every other row is
    // considered by exactly one thread, so nothing else can be there twice
    if (__ldcg(d.cand_rows + (size_t)mu * CAND_CAP) == row) return;
    const int slot = atomicAdd(d.cand_n + mu, 1);
    if (slot < CAND_CAP) d.cand_rows[(size_t)mu * CAND_CAP + slot] = row;
    else atomicMax(d.cand_floor + mu, u);
  };
  for (int row = blockIdx.x * groups + g; row < nrows; row += SCAN_UNROLL * stride) {
    uint4 v[SCAN_UNROLL];
#pragma unroll
    for (int u = 0; u < SCAN_UNROLL; ++u) {
      const int rr = row + u * stride;
      v[u] = __ldcg(base + (size_t)(radd + rmul * (rr < nrows ? rr : row)) * Kq);
    }
#pragma unroll
    for (int u = 0; u < SCAN_UNROLL; ++u) {
      const int rr = row + u * stride;
      if (rr >= nrows) continue;
      const int r = radd + rmul * rr;
      consider(v[u].x, 0, r);
      consider(v[u].y, 1, r);
      consider(v[u].z, 2, r);
      consider(v[u].w, 3, r);
    }
  }
}

// ---------------------------------------------------------------------------
// T12 + T13.  Every CTA derives nc and the step size from the K column maxima
// (cheap) and then walks its share of the slots: owners write
//   wt = parked + cnt * f_i * s / (n * alpha')     with alpha' = alpha * (1 - s*X)
// and clear their count.  CTA 0 publishes alpha' and the step's nc and s, and
// clears the maxima the next step will accumulate into.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256) k_apply(Dev d, int local, const int32_t* __restrict__ idx) {
  grid_dependency_wait();
  if (blockIdx.x == 0 && threadIdx.x == 0) phase_mark(d.ctl, PH_APPLY);
  if (d.ctl->error & FV_DEVERR_TIMEOUT) return;  // a peer never answered: the step loop is void
  extern __shared__ __align__(16) unsigned char smem_raw[];
  double* sX = reinterpret_cast<double*>(smem_raw);  // mean xx over active ranks, later s / (n * alpha')
  int* sN = reinterpret_cast<int*>(sX + d.Kp);
  uint32_t* sFloor = reinterpret_cast<uint32_t*>(sN + d.Kp);  // the units' candidate floors as this kernel found them
  __shared__ float sRed[8];
  __shared__ float sScale;
  const int p = (int)((d.tick0 + local) & 1);
  const double* __restrict__ alpha = d.alpha + p * d.Kp;
  double* __restrict__ alpha_next = d.alpha + (p ^ 1) * d.Kp;

  float dense = 0.f;
  for (int mu = threadIdx.x; mu < d.Kp; mu += blockDim.x) {
    const double X = d.stat_x[p * d.Kp + mu];  // left by the scan kernel
    const int n = d.stat_n[p * d.Kp + mu];
    sFloor[mu] = d.use_cand ? __ldcg(d.cand_floor + mu) : 0xffffffffu;  // final since the previous kernel; it can only rise here
    sX[mu] = X;
    sN[mu] = n;
    if (n > 0) dense = fmaxf(dense, (float)(fabs(X * alpha[mu]) * (double)__uint_as_float(d.colmax[p * d.Kp + mu])));
  }
  dense = warp_max(dense);
  if ((threadIdx.x & 31) == 0) sRed[threadIdx.x >> 5] = dense;
  __syncthreads();
  __shared__ int sFail;
  if (threadIdx.x == 0) sFail = 0;
  __syncthreads();
  const unsigned seq = (unsigned)(d.tick0 + local + 1);
  __shared__ uint32_t sWord[MAX_RANKS];
  __shared__ uint32_t sCount[MAX_RANKS];
  if (d.shard && threadIdx.x < d.G) {
    // every rank's partial normaliser (pushed by its k_scan) must have arrived, ours included,
    // and with it the length of its entry list
    const unsigned long long* words = reinterpret_cast<const unsigned long long*>(d.mail + WORD_NC);
    if (!wait_word(d, words + p * MAX_RANKS + threadIdx.x, seq, &sWord[threadIdx.x])) sFail = 1;
    const unsigned long long* outw = reinterpret_cast<const unsigned long long*>(d.mail + WORD_OUT);
    if (!wait_word(d, outw + p * MAX_RANKS + threadIdx.x, seq, &sCount[threadIdx.x])) sFail = 1;
  }
  __syncthreads();
  if (sFail) return;
  if (threadIdx.x == 0) {
    float nc = 0.f;
    if (d.shard) {
      for (int r = 0; r < d.G; ++r) nc = fmaxf(nc, __uint_as_float(sWord[r]));
    } else {
      nc = __uint_as_float(d.ncb[p]);
      for (int w = 0; w < (int)(blockDim.x >> 5); ++w) nc = fmaxf(nc, sRed[w]);
    }
    const float eps = d.ctl->eps;
    const float s = (d.prec > nc) ? eps / d.prec : eps / nc;  // cuda_funcs.cu:1797-1799
    sScale = s;
    if (blockIdx.x == 0) {
      d.nc_log[local] = nc;
      d.s_log[local] = s;
    }
  }
  __syncthreads();
  const float s = sScale;
  for (int mu = threadIdx.x; mu < d.Kp; mu += blockDim.x) {
    const int n = sN[mu];
    double a = alpha[mu];
    double coef = 0.0;
    if (n > 0) {
      a = a * (1.0 - (double)s * sX[mu]);
      if (a != 0.0)
        coef = (double)s / ((double)n * a);
      else
        atomicOr(&d.ctl->error, FV_DEVERR_NAN_WEIGHT);
    }
    sX[mu] = coef;
    if (blockIdx.x == 0) {
      alpha_next[mu] = a;
      d.colmax[(p ^ 1) * d.Kp + mu] = 0u;
    }
  }
  if (blockIdx.x == 0 && threadIdx.x == 0) d.ncb[p ^ 1] = 0u;
  __syncthreads();

  uint32_t vmax = 0u;
  const int nrec = (int)min(d.ctl->list_count[p], (uint32_t)d.rec_cap);
  const float delta = d.ctl->delta;
  if (blockIdx.x == 0 && threadIdx.x == 0) d.ctl->list_count[p ^ 1] = 0u;  // the next step counts from zero
  const int nthreads = gridDim.x * blockDim.x;
  const int gtid = blockIdx.x * blockDim.x + threadIdx.x;
  {
    // this rank's records: the parked weight comes back with its scatter term
    constexpr int UN = 4;
    for (int k0 = gtid; k0 < nrec; k0 += UN * nthreads) {
      int cp[UN], cn[UN];
      uint4 r[UN];
#pragma unroll
      for (int u = 0; u < UN; ++u) {
        const int k = k0 + u * nthreads;
        cp[u] = (k < nrec) ? d.cnt[k] : 0;
        cn[u] = (k < nrec && d.has_delta) ? d.cntn[k] : 0;
        r[u] = (k < nrec) ? d.rec[k] : make_uint4(0u, 0u, 0u, 0u);
      }
#pragma unroll
      for (int u = 0; u < UN; ++u) {
        if (r[u].w == 0u) continue;  // a hole
        const int k = k0 + u * nthreads;
        const int mu = (int)(r[u].x % (uint32_t)d.Kp);
        const double scat = (double)(cp[u] + (int)(r[u].w & 0xffffu)) - (double)delta * (double)(cn[u] + (int)(r[u].w >> 16));
        const float v = (float)((double)__uint_as_float(r[u].y) + scat * (double)__uint_as_float(r[u].z) * sX[mu]);
        d.wt[r[u].x] = v;
        d.rec[k].w = 0u;  // the slot is a hole again until it is claimed anew
        if (cp[u]) d.cnt[k] = 0;
        if (cn[u]) d.cntn[k] = 0;
        const uint32_t vb = __float_as_uint(fabsf(v));
        vmax = max(vmax, vb);
        if (vb > sFloor[mu] && vb > __ldcg(d.cand_floor + mu)) {
          // the new weight rises above its unit's floor: list its row, or lift the floor when the list is full
          const int irow = (int)(r[u].x / (uint32_t)d.Kp);
          const int n = min(__ldcg(d.cand_n + mu), CAND_CAP);
          bool have = false;
          for (int j = 0; j < n; ++j) have |= (__ldcg(d.cand_rows + (size_t)mu * CAND_CAP + j) == irow);
          if (!have) {
            const int slot = atomicAdd(d.cand_n + mu, 1);
            if (slot < CAND_CAP) d.cand_rows[(size_t)mu * CAND_CAP + slot] = irow;
            else atomicMax(d.cand_floor + mu, vb);
          }
        }
      }
    }
  }
  if (d.shard) {
    // the rows owned elsewhere: the same arithmetic on this replica's copy of the weight, with the
    // count the owner sent (the owner's parked weight and this copy are the same number)
    constexpr int UN = 4;
    const uint32_t limit = (uint32_t)((size_t)d.N * d.Kp);
    for (int r = 0; r < d.G; ++r) {
      if (r == d.rank) continue;
      const int n_r = (int)min(sCount[r], (uint32_t)d.inbox_cap);
      unsigned long long* __restrict__ box = inbox(d, d.mail, r);
      for (int k0 = gtid; k0 < n_r; k0 += UN * nthreads) {
        unsigned long long e[UN];
#pragma unroll
        for (int u = 0; u < UN; ++u) {
          const int k = k0 + u * nthreads;
          e[u] = (k < n_r) ? load_relaxed_sys64(box + k) : (unsigned long long)ENTRY_HOLE;
        }
        uint32_t w_old[UN];
#pragma unroll
        for (int u = 0; u < UN; ++u) {
          const int k = k0 + u * nthreads;
          if (!((uint32_t)e[u] & ENTRY_VALID)) {  // still on its way (bounded wait)
            unsigned polls = 0;
            for (;;) {
              e[u] = load_relaxed_sys64(box + k);
              if ((uint32_t)e[u] & ENTRY_VALID) break;
              if (wait_expired(d, polls)) {
                e[u] = (unsigned long long)ENTRY_HOLE;
                break;
              }
            }
          }
          const uint32_t lo = (uint32_t)e[u];
          w_old[u] = 0u;
          if (lo != ENTRY_HOLE) {
            if ((lo & ~ENTRY_VALID) < limit) {
              w_old[u] = __ldcg(reinterpret_cast<const uint32_t*>(d.wt) + (lo & ~ENTRY_VALID));
            } else {
              atomicOr(&d.ctl->error, FV_DEVERR_SLOT_RANGE);
              e[u] = (unsigned long long)ENTRY_HOLE;
            }
          }
        }
#pragma unroll
        for (int u = 0; u < UN; ++u) {
          const int k = k0 + u * nthreads;
          if (k >= n_r) continue;
          box[k] = 0ull;  // used
          const uint32_t lo = (uint32_t)e[u];
          if (lo == ENTRY_HOLE) continue;
          const uint32_t pos = lo & ~ENTRY_VALID;
          const int irow = (int)fdiv(pos, d.mKp, d.sKp);
          const int mu = (int)pos - irow * d.Kp;
          const double scat = (double)(int)(uint32_t)(e[u] >> 32);
          const float f = __ldg(d.f + (irow >= d.V ? irow - d.V : irow));
          const float v = (float)((double)__uint_as_float(w_old[u]) + scat * (double)f * sX[mu]);
          d.wt[pos] = v;
          vmax = max(vmax, __float_as_uint(fabsf(v)));
        }
      }
    }
  }
  // keep the bound on max |wt| valid for the next forward pass
  vmax = warp_max_u32(vmax);
  if ((threadIdx.x & 31) == 0 && vmax > d.ctl->wabsmax) atomicMax(&d.ctl->wabsmax, vmax);
}

// ---------------------------------------------------------------------------
// k_eval and k_apply as ONE kernel for ordinary steps (no list rebuild, replicated or single-rank update).
// Both halves are short chains of dependent accesses and the second needs only two things of the first
// grid-wide -- the largest |D| at the records and the units' column maxima -- so the grid meets once at a
// counter instead of ending and starting again: one launch less per step, and a record CTA keeps the
// records it evaluated in registers and applies them without loading them a second time.
//   CTAs [0, qblocks)   query the candidate lists (as in k_eval), then help nobody: they are done
//   the other CTAs      evaluate D at their records, meet, derive nc and the step size, apply their records
// The meeting point is a 64-bit arrival counter that only grows (`target` = the count once all CTAs of this
// launch are in; the host counts the launches), so nothing has to be reset; every CTA of the grid is resident (the launch is sized by the occupancy calculator), the wait is
// bounded like every other wait here.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(SCAN_THREADS, 2) k_update(Dev d, int local, const int32_t* __restrict__ idx, int qblocks,
                                                            unsigned long long target) {
  grid_dependency_wait();
  if (blockIdx.x == 0 && threadIdx.x == 0) phase_mark(d.ctl, PH_SCAN);
  if (d.ctl->error & FV_DEVERR_TIMEOUT) return;  // a peer never answered: the step loop is void
  const int p = (int)((d.tick0 + local) & 1);
  const int lane = threadIdx.x & 31;
  const uint32_t seq = (uint32_t)(d.tick0 + local + 1);
  __shared__ int s_fail;
  if (threadIdx.x == 0) s_fail = 0;

  // ---- first half ---------------------------------------------------------------------------------
  constexpr int TS = 4;
  int cp[TS], cn[TS];
  uint4 rc[TS];
  extern __shared__ __align__(16) unsigned char smem_raw[];
  double* sC = reinterpret_cast<double*>(smem_raw);                // X*alpha, later s / (n * alpha')
  double* sXm = sC + d.Kp;                                         // mean xx over the active ranks
  int* sN = reinterpret_cast<int*>(sXm + d.Kp);                    // active ranks
  uint32_t* sBad = reinterpret_cast<uint32_t*>(sN + d.Kp);         // ranks whose windows must leave the counts
  uint32_t* sFloor = sBad + d.Kp;                                  // the units' candidate floors
  double* sAl = reinterpret_cast<double*>(sFloor + d.Kp);          // the units' scales (Kp is a multiple of 4: aligned)
  const bool query_cta = (int)blockIdx.x < qblocks;
  const int nrec = (int)min(d.ctl->list_count[p], (uint32_t)d.rec_cap);
  const int nthreads = (gridDim.x - qblocks) * blockDim.x;
  const int e0 = ((int)blockIdx.x - qblocks) * (int)blockDim.x + (int)threadIdx.x;
  const float delta = d.ctl->delta;
  const float eps = d.ctl->eps;

  if (query_cta) {
    constexpr int QW = SCAN_THREADS / 32;
    __shared__ int s_unc[QW];
    const int wic = threadIdx.x >> 5;
    const int mu = blockIdx.x * QW + wic;
    if (lane == 0) s_unc[wic] = 0;
    if (mu < d.K) {
      const uint32_t* __restrict__ wbits = reinterpret_cast<const uint32_t*>(d.wt);
      const int n = min(__ldcg(d.cand_n + mu), CAND_CAP);
      const uint32_t floor_bits = __ldcg(d.cand_floor + mu);
      int row[CAND_CAP / 32];
#pragma unroll
      for (int t = 0; t < CAND_CAP / 32; ++t) row[t] = (lane + 32 * t < n) ? __ldcg(d.cand_rows + (size_t)mu * CAND_CAP + lane + 32 * t) : -1;
      uint32_t xbits = 0u;
      if (lane < d.G) {
        const unsigned long long* word = packet(d, p, lane) + d.XO + mu;
        const unsigned long long w = load_relaxed_sys64(word);
        xbits = ((uint32_t)(w >> 32) == seq) ? (uint32_t)w : pk_read(d, word, seq, 0u);
      }
      const bool active = __any_sync(FULL, lane < d.G && __uint_as_float(xbits) != 0.f);
      if (active) {
        uint32_t m = 0u;
#pragma unroll
        for (int t = 0; t < CAND_CAP / 32; ++t) {
          if (row[t] < 0) continue;
          const uint32_t w = __ldcg(wbits + (size_t)row[t] * d.Kp + mu) & ABS_MASK;
          m = max(m, w > TAG_BASE ? 0u : w);
        }
        m = warp_max_u32(m);
        if (lane == 0) {
          if (m >= floor_bits) d.colmax[p * d.Kp + mu] = m;
          else s_unc[wic] = 1;
        }
      }
    }
    __syncthreads();
    for (int w = 0; w < QW; ++w) {
      if (!s_unc[w]) continue;
      // every strong candidate of this unit was touched: read its whole column (see k_eval)
      const int cu = blockIdx.x * QW + w;
      const uint32_t* __restrict__ col = reinterpret_cast<const uint32_t*>(d.wt) + cu;
      unsigned long long best = 0ull;
      constexpr int RU = 8;
      for (int r0 = threadIdx.x; r0 < d.N; r0 += RU * SCAN_THREADS) {
        uint32_t v[RU];
#pragma unroll
        for (int u = 0; u < RU; ++u) {
          const int r = r0 + u * SCAN_THREADS;
          v[u] = (r < d.N) ? (__ldcg(col + (size_t)r * d.Kp) & ABS_MASK) : 0u;
        }
#pragma unroll
        for (int u = 0; u < RU; ++u) {
          const int r = r0 + u * SCAN_THREADS;
          if (r < d.N && v[u] <= TAG_BASE) best = max(best, ((unsigned long long)v[u] << 32) | (uint32_t)r);
        }
      }
#pragma unroll
      for (int o = 16; o >= 1; o >>= 1) best = max(best, __shfl_xor_sync(FULL, best, o));
      __shared__ unsigned long long s_best[QW];
      if (lane == 0) s_best[wic] = best;
      __syncthreads();
      if (threadIdx.x == 0) {
        for (int k = 1; k < QW; ++k) best = max(best, s_best[k]);
        const uint32_t m = (uint32_t)(best >> 32);
        d.colmax[p * d.Kp + cu] = m;
        d.cand_floor[cu] = m;
        if (m) {
          const int row = (int)(uint32_t)best;
          const int n = min(d.cand_n[cu], CAND_CAP);
          bool have = false;
          for (int j = 0; j < n; ++j) have |= (d.cand_rows[(size_t)cu * CAND_CAP + j] == row);
          if (!have) {
            const int slot = (n < CAND_CAP) ? n : (int)((d.tick0 + local + (unsigned)cu) % CAND_CAP);
            d.cand_rows[(size_t)cu * CAND_CAP + slot] = row;
            d.cand_n[cu] = (n < CAND_CAP) ? n + 1 : CAND_CAP;
          } else {
            d.cand_n[cu] = n;
          }
        }
        atomicAdd(&d.ctl->scans_run, 1u);
      }
      __syncthreads();
    }
  } else {
    const double* __restrict__ alpha = d.alpha + p * d.Kp;
    __shared__ int s_any_bad;
    auto load_batch = [&](int k0) {
#pragma unroll
      for (int u = 0; u < TS; ++u) {
        const int k = k0 + u * nthreads;
        cp[u] = (k < nrec) ? d.cnt[k] : 0;
        cn[u] = (k < nrec && d.has_delta) ? d.cntn[k] : 0;
        rc[u] = (k < nrec) ? d.rec[k] : make_uint4(0u, 0u, 0u, 0u);
      }
    };
    load_batch(e0);  // in flight while the combine below polls the packets
    if (threadIdx.x == 0) s_any_bad = 0;
    __syncthreads();
    for (int mu = threadIdx.x; mu < d.Kp; mu += blockDim.x) {
      double X = 0.0;
      int n = 0;
      if (mu < d.K) unit_stats(d, p, seq, mu, &X, &n);
      const double al = alpha[mu];
      sAl[mu] = al;
      sC[mu] = X * al;
      sXm[mu] = X;
      sN[mu] = n;
      const uint32_t bad = (mu < d.K && n > 0) ? unit_cancelled(d, p, mu) : 0u;
      sBad[mu] = bad;
      if (bad) s_any_bad = 1;
    }
    __syncthreads();
    if (s_any_bad) {
      const unsigned long long* packet0 = packet(d, p, 0);
      for (int k = e0; k < nrec; k += nthreads) {
        const uint4 r = d.rec[k];
        if (r.w == 0u) continue;
        const int irow = (int)fdiv(r.x, d.mKp, d.sKp);
        const int mu = (int)r.x - irow * d.Kp;
        if (!sBad[mu]) continue;
        const int2 c = cancelled_multiplicity(packet0, d.P, d.G, d.B, d.W, d.MO, d.has_delta, idx, d.idx_rstride, irow, mu, sBad[mu]);
        if (c.x) d.cnt[k] -= c.x;
        if (c.y) d.cntn[k] -= c.y;
      }
      load_batch(e0);  // the counts have changed
    }
    uint32_t tmax = 0u;
    auto eval_batch = [&]() {
#pragma unroll
      for (int u = 0; u < TS; ++u) {
        if (rc[u].w == 0u) continue;  // a hole (or past the end)
        const int mu = (int)(rc[u].x - fdiv(rc[u].x, d.mKp, d.sKp) * (uint32_t)d.Kp);
        if (sN[mu] == 0) continue;
        const float c = (float)(cp[u] + (int)(rc[u].w & 0xffffu)) - delta * (float)(cn[u] + (int)(rc[u].w >> 16));
        const double D = -sC[mu] * (double)__uint_as_float(rc[u].y) + (double)c * (double)__uint_as_float(rc[u].z) / (double)sN[mu];
        tmax = max(tmax, __float_as_uint(fabsf((float)D)));
      }
    };
    eval_batch();
    for (int k0 = e0 + TS * nthreads; k0 < nrec; k0 += TS * nthreads) {  // more records than one batch per thread (many ranks)
      load_batch(k0);
      eval_batch();
    }
    if (e0 + TS * nthreads < nrec) load_batch(e0);  // back to the first batch for the second half
    __shared__ uint32_t s_tmax;
    if (threadIdx.x == 0) s_tmax = 0u;
    __syncthreads();
    tmax = warp_max_u32(tmax);
    if (lane == 0 && tmax) atomicMax(&s_tmax, tmax);
    __syncthreads();
    if (threadIdx.x == 0 && s_tmax) atomicMax(&d.ncb[p], s_tmax);
  }

  // ---- the grid meets -------------------------------------------------------------------------------
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    atomicAdd(&d.ctl->update_arrivals, 1ull);
    // (the failure flag of another wait is looked at every 64th poll only: one load per poll keeps the
    // meeting point's latency at one L2 round trip)
    unsigned polls = 0;
    while (*reinterpret_cast<volatile unsigned long long*>(&d.ctl->update_arrivals) < target) {
      if ((++polls & 63u) == 0u) {
        if (polls > d.spin_limit || (*reinterpret_cast<volatile uint32_t*>(&d.ctl->error) & FV_DEVERR_TIMEOUT)) {
          atomicOr(&d.ctl->error, FV_DEVERR_TIMEOUT);
          s_fail = 1;
          break;
        }
        if (polls > 4096u) __nanosleep(128);
      }
    }
    __threadfence();
    if ((int)blockIdx.x == qblocks) phase_mark(d.ctl, PH_APPLY);  // the clock's "apply" is the second half as this CTA sees it
  }
  __syncthreads();
  if (s_fail || query_cta) return;

  // ---- second half: normaliser, step size, the records come back with their scatter term ------------
  double* __restrict__ alpha_next = d.alpha + (p ^ 1) * d.Kp;
  __shared__ float sRed[SCAN_THREADS / 32];
  __shared__ float sScale;
  const bool first = (int)blockIdx.x == qblocks;  // the CTA that writes what there is one of
  // everything the second half reads from memory leaves together: the maxima, the floors, the records' maximum
  const uint32_t ncb_bits = (threadIdx.x == 0) ? __ldcg(&d.ncb[p]) : 0u;
  float dense = 0.f;
  for (int mu = threadIdx.x; mu < d.Kp; mu += blockDim.x) {
    sFloor[mu] = __ldcg(d.cand_floor + mu);
    if (sN[mu] > 0) dense = fmaxf(dense, (float)(fabs(sC[mu]) * (double)__uint_as_float(__ldcg(&d.colmax[p * d.Kp + mu]))));
  }
  dense = warp_max(dense);
  if (lane == 0) sRed[threadIdx.x >> 5] = dense;
  __syncthreads();
  if (threadIdx.x == 0) {
    float nc = __uint_as_float(ncb_bits);
    for (int w = 0; w < SCAN_THREADS / 32; ++w) nc = fmaxf(nc, sRed[w]);
    const float s = (d.prec > nc) ? eps / d.prec : eps / nc;  // cuda_funcs.cu:1797-1799
    sScale = s;
    if (first) {
      d.nc_log[local] = nc;
      d.s_log[local] = s;
    }
  }
  __syncthreads();
  const float s = sScale;
  for (int mu = threadIdx.x; mu < d.Kp; mu += blockDim.x) {
    const int n = sN[mu];
    double a = sAl[mu];
    double coef = 0.0;
    if (n > 0) {
      a = a * (1.0 - (double)s * sXm[mu]);
      if (a != 0.0)
        coef = (double)s / ((double)n * a);
      else
        atomicOr(&d.ctl->error, FV_DEVERR_NAN_WEIGHT);
    }
    sC[mu] = coef;
    if (first) {
      alpha_next[mu] = a;
      d.stat_x[p * d.Kp + mu] = sXm[mu];
      d.stat_n[p * d.Kp + mu] = n;
    }
  }
  __syncthreads();
  uint32_t vmax = 0u;
  auto apply_batch = [&](int k0) {
#pragma unroll
    for (int u = 0; u < TS; ++u) {
      if (rc[u].w == 0u) continue;  // a hole
      const int k = k0 + u * nthreads;
      const int mu = (int)(rc[u].x - fdiv(rc[u].x, d.mKp, d.sKp) * (uint32_t)d.Kp);
      const double scat = (double)(cp[u] + (int)(rc[u].w & 0xffffu)) - (double)delta * (double)(cn[u] + (int)(rc[u].w >> 16));
      const float v = (float)((double)__uint_as_float(rc[u].y) + scat * (double)__uint_as_float(rc[u].z) * sC[mu]);
      d.wt[rc[u].x] = v;
      d.rec[k].w = 0u;  // the slot is a hole again until it is claimed anew
      if (cp[u]) d.cnt[k] = 0;
      if (cn[u]) d.cntn[k] = 0;
      const uint32_t vb = __float_as_uint(fabsf(v));
      vmax = max(vmax, vb);
      if (vb > sFloor[mu] && vb > __ldcg(d.cand_floor + mu)) {
        // the new weight rises above its unit's floor: list its row, or lift the floor when the list is full
        const int irow = (int)fdiv(rc[u].x, d.mKp, d.sKp);
        const int n = min(__ldcg(d.cand_n + mu), CAND_CAP);
        bool have = false;
        for (int j = 0; j < n; ++j) have |= (__ldcg(d.cand_rows + (size_t)mu * CAND_CAP + j) == irow);
        if (!have) {
          const int slot = atomicAdd(d.cand_n + mu, 1);
          if (slot < CAND_CAP) d.cand_rows[(size_t)mu * CAND_CAP + slot] = irow;
          else atomicMax(d.cand_floor + mu, vb);
        }
      }
    }
  };
  apply_batch(e0);
  for (int k0 = e0 + TS * nthreads; k0 < nrec; k0 += TS * nthreads) {
#pragma unroll
    for (int u = 0; u < TS; ++u) {
      const int k = k0 + u * nthreads;
      cp[u] = (k < nrec) ? d.cnt[k] : 0;
      cn[u] = (k < nrec && d.has_delta) ? d.cntn[k] : 0;
      rc[u] = (k < nrec) ? d.rec[k] : make_uint4(0u, 0u, 0u, 0u);
    }
    apply_batch(k0);
  }
  // keep the bound on max |wt| valid for the next forward pass
  vmax = warp_max_u32(vmax);
  if (lane == 0 && vmax > d.ctl->wabsmax) atomicMax(&d.ctl->wabsmax, vmax);
  // what the next step must find cleared (no CTA reads these again in this step: all are past the meeting point)
  if (first) {
    for (int mu = threadIdx.x; mu < d.Kp; mu += blockDim.x) d.colmax[(p ^ 1) * d.Kp + mu] = 0u;
    if (threadIdx.x == 0) {
      d.ncb[p ^ 1] = 0u;
      d.ctl->list_count[p ^ 1] = 0u;
    }
  }
}

// ---------------------------------------------------------------------------
// Folding the scale into the weights: wt[i][mu] *= alpha[mu]; then alpha = 1.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256) k_fold(Dev d, int local) {
  grid_dependency_wait();
  if (blockIdx.x == 0 && threadIdx.x == 0) phase_mark(d.ctl, PH_FOLD);
  // `local` = steps already launched in this call: the buffer the next step would read
  const double* __restrict__ alpha = d.alpha + ((d.tick0 + local) & 1) * d.Kp;
  const size_t total = (size_t)d.N * d.Kq;
  float vmax = 0.f;
  for (size_t v = (size_t)blockIdx.x * blockDim.x + threadIdx.x; v < total; v += (size_t)gridDim.x * blockDim.x) {
    const int q = (int)(v % d.Kq);
    float4* ptr = reinterpret_cast<float4*>(d.wt) + v;
    float4 x = *ptr;
    x.x = (float)((double)x.x * alpha[4 * q + 0]);
    x.y = (float)((double)x.y * alpha[4 * q + 1]);
    x.z = (float)((double)x.z * alpha[4 * q + 2]);
    x.w = (float)((double)x.w * alpha[4 * q + 3]);
    *ptr = x;
    vmax = fmaxf(vmax, fmaxf(fmaxf(fabsf(x.x), fabsf(x.y)), fmaxf(fabsf(x.z), fabsf(x.w))));
  }
  vmax = warp_max(vmax);
  if ((threadIdx.x & 31) == 0) atomicMax(&d.ctl->wabsmax_fold, __float_as_uint(vmax));
}
// Runs after k_fold or after new weights were loaded; both collect max |wt| in wabsmax_fold.
__global__ void k_reset_alpha(Dev d) {
  grid_dependency_wait();
  // both buffers become 1, so the parity of the next step does not matter
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < 2 * d.Kp; i += gridDim.x * blockDim.x) d.alpha[i] = 1.0;
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    d.ctl->wabsmax = d.ctl->wabsmax_fold;
    d.ctl->wabsmax_fold = 0u;
  }
}
__global__ void k_absmax(Dev d) {
  const size_t total = (size_t)d.N * d.Kp;
  float vmax = 0.f;
  for (size_t v = (size_t)blockIdx.x * blockDim.x + threadIdx.x; v < total; v += (size_t)gridDim.x * blockDim.x)
    vmax = fmaxf(vmax, fabsf(d.wt[v]));
  vmax = warp_max(vmax);
  if ((threadIdx.x & 31) == 0) atomicMax(&d.ctl->wabsmax_fold, __float_as_uint(vmax));
}

// ---------------------------------------------------------------------------
// Layout changes between the checkpoint layout [K][N] and wt [N][Kp].
// ---------------------------------------------------------------------------
__global__ void k_to_device_layout(const float* __restrict__ w_kn, float* __restrict__ wt, int K, int Kp, int N) {
  __shared__ float tile[32][33];
  const int i0 = blockIdx.x * 32, m0 = blockIdx.y * 32;
  for (int r = threadIdx.y; r < 32; r += blockDim.y) {
    const int mu = m0 + r, i = i0 + threadIdx.x;
    tile[r][threadIdx.x] = (mu < K && i < N) ? w_kn[(size_t)mu * N + i] : 0.f;
  }
  __syncthreads();
  for (int r = threadIdx.y; r < 32; r += blockDim.y) {
    const int i = i0 + r, mu = m0 + threadIdx.x;
    if (i < N && mu < Kp) wt[(size_t)i * Kp + mu] = tile[threadIdx.x][r];
  }
}
__global__ void k_to_host_layout(const float* __restrict__ wt, float* __restrict__ w_kn, int K, int Kp, int N) {
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

// ---------------------------------------------------------------------------
// Seeded window order: a keyed bijection of [0, n) (balanced Feistel network on
// 2*half bits, cycle-walked into range), evaluated independently per index.
// ---------------------------------------------------------------------------
__device__ __forceinline__ uint32_t mix32(uint32_t x, uint32_t k) {
  x ^= k;
  x *= 0x85ebca6bu;
  x ^= x >> 13;
  x *= 0xc2b2ae35u;
  x ^= x >> 16;
  return x;
}
__global__ void k_feistel_perm(unsigned long long* __restrict__ perm, unsigned long long n, int half,
                               unsigned long long seed) {
  const unsigned long long mask = (1ull << half) - 1ull;
  for (unsigned long long i = (unsigned long long)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (unsigned long long)gridDim.x * blockDim.x) {
    unsigned long long x = i;
    do {
      uint32_t L = (uint32_t)(x >> half), R = (uint32_t)(x & mask);
#pragma unroll
      for (int r = 0; r < 6; ++r) {
        const uint32_t k = (uint32_t)(seed >> ((r & 1) * 32)) + 0x9e3779b9u * (uint32_t)(r + 1);
        const uint32_t F = mix32(R, k) & (uint32_t)mask;
        const uint32_t nl = R;
        R = L ^ F;
        L = nl;
      }
      x = ((unsigned long long)L << half) | R;
    } while (x >= n);
    perm[i] = x;
  }
}
__global__ void k_iota(unsigned long long* __restrict__ perm, unsigned long long n) {
  for (unsigned long long i = (unsigned long long)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (unsigned long long)gridDim.x * blockDim.x)
    perm[i] = i;
}

// ---------------------------------------------------------------------------
// Corpus preparation on the GPU (T1: prune_input.cpp:63-122, T2: model_arrays.cu:395-424).
//   k_chunk_windows   windows per chunk: len - w + 1 when w <= len < maxlen, else 0
//   k_block_scan      exclusive prefix of those counts, 1024 chunks per CTA (the CTA totals are
//                     prefixed on the host: a few thousand numbers)
//   k_fill_starts     one thread per window: binary search for its chunk, start = running sum of
//                     the chunk lengths before it (= offsets[s] - offsets[0]) + position in the chunk
//   k_count_tokens    histogram of the token ids: per-CTA shared-memory bins when the vocabulary
//                     fits, merged with 64-bit atomics; ids >= V raise the device error word
//   k_inverse_counts  f[v] = (float)(1.0 / count), 0 for unseen ids, counts capped at 2^24 on request
// ---------------------------------------------------------------------------
__global__ void k_chunk_windows(const unsigned long long* __restrict__ off, unsigned long long nchunks, unsigned W,
                                unsigned maxlen, uint32_t* __restrict__ nwin, uint32_t* error) {
  for (unsigned long long s = (unsigned long long)blockIdx.x * blockDim.x + threadIdx.x; s < nchunks;
       s += (unsigned long long)gridDim.x * blockDim.x) {
    const unsigned long long a = off[s], b = off[s + 1];
    uint32_t n = 0;
    if (b < a) {
      atomicOr(error, FV_DEVERR_WINDOW_RANGE);
    } else {
      const unsigned long long len = b - a;
      if (len >= W && len < maxlen) n = (uint32_t)(len - W + 1);
    }
    nwin[s] = n;
  }
}
constexpr int SCAN_BLOCK = 1024;
__global__ void __launch_bounds__(SCAN_BLOCK) k_block_scan(const uint32_t* __restrict__ nwin, unsigned long long nchunks,
                                                           const unsigned long long* __restrict__ block_base,
                                                           unsigned long long* __restrict__ wbase,
                                                           unsigned long long* __restrict__ block_total) {
  __shared__ unsigned long long s_w[SCAN_BLOCK / 32];
  const unsigned long long s = (unsigned long long)blockIdx.x * SCAN_BLOCK + threadIdx.x;
  const unsigned long long v = (s < nchunks) ? nwin[s] : 0ull;
  unsigned long long incl = v;
  const int lane = threadIdx.x & 31, wic = threadIdx.x >> 5;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const unsigned long long t = __shfl_up_sync(FULL, incl, o);
    if (lane >= o) incl += t;
  }
  if (lane == 31) s_w[wic] = incl;
  __syncthreads();
  if (wic == 0) {
    unsigned long long t = s_w[lane];
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const unsigned long long u = __shfl_up_sync(FULL, t, o);
      if (lane >= o) t += u;
    }
    s_w[lane] = t;  // inclusive prefix of the warp totals
  }
  __syncthreads();
  const unsigned long long before = (wic ? s_w[wic - 1] : 0ull) + incl - v;
  if (block_base) {
    if (s < nchunks) wbase[s] = block_base[blockIdx.x] + before;
  } else if (threadIdx.x == SCAN_BLOCK - 1) {
    block_total[blockIdx.x] = before + v;
  }
}
__global__ void k_fill_starts(const unsigned long long* __restrict__ off, const unsigned long long* __restrict__ wbase,
                              unsigned long long nchunks, unsigned long long ns, unsigned long long* __restrict__ starts) {
  const unsigned long long origin = off[0];
  for (unsigned long long p = (unsigned long long)blockIdx.x * blockDim.x + threadIdx.x; p < ns;
       p += (unsigned long long)gridDim.x * blockDim.x) {
    // last chunk s with wbase[s] <= p (chunks without windows share their successor's base and are skipped)
    unsigned long long lo = 0, hi = nchunks;
    while (hi - lo > 1) {
      const unsigned long long mid = (lo + hi) >> 1;
      if (wbase[mid] <= p) lo = mid; else hi = mid;
    }
    starts[p] = (off[lo] - origin) + (p - wbase[lo]);
  }
}
__global__ void __launch_bounds__(512) k_count_tokens(const int32_t* __restrict__ tok, unsigned long long n, int V,
                                                      int use_smem, unsigned long long* __restrict__ counts,
                                                      uint32_t* error) {
  extern __shared__ uint32_t s_bins[];
  if (use_smem) {
    for (int v = threadIdx.x; v < V; v += blockDim.x) s_bins[v] = 0u;
    __syncthreads();
  }
  for (unsigned long long i = (unsigned long long)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (unsigned long long)gridDim.x * blockDim.x) {
    const int t = tok[i];
    if (t < 0) continue;  // negative ids are padding and do not count (model_arrays.cu:414)
    if (t >= V) {
      atomicOr(error, FV_DEVERR_TOKEN_RANGE);
      continue;
    }
    if (use_smem) atomicAdd(&s_bins[t], 1u); else atomicAdd(&counts[t], 1ull);
  }
  if (use_smem) {
    __syncthreads();
    for (int v = threadIdx.x; v < V; v += blockDim.x)
      if (s_bins[v]) atomicAdd(&counts[v], (unsigned long long)s_bins[v]);
  }
}
// The HOT_TOKENS most frequent tokens (smallest positive 1/count; ties by id) and the hot-row numbers of their
// context row (token) and target row (V + token).  One CTA; `picked` receives the number of hot rows.
__global__ void __launch_bounds__(1024) k_pick_hot(const float* __restrict__ f, int V, int8_t* __restrict__ hotidx,
                                                   int32_t* __restrict__ hot_rows, int* __restrict__ picked) {
  __shared__ unsigned long long s_best[32];
  __shared__ unsigned long long s_last;
  const int lane = threadIdx.x & 31, wic = threadIdx.x >> 5;
  if (threadIdx.x == 0) s_last = 0ull;
  __syncthreads();
  int n = 0;
  for (int h = 0; h < HOT_TOKENS; ++h) {
    const unsigned long long last = s_last;
    unsigned long long best = ~0ull;  // key = (bits of 1/count, id): the smallest key above the last pick
    for (int v = threadIdx.x; v < V; v += blockDim.x) {
      const float x = f[v];
      if (!(x > 0.f)) continue;
      const unsigned long long key = ((unsigned long long)__float_as_uint(x) << 32) | (unsigned)(v + 1);
      if (key > last && key < best) best = key;
    }
#pragma unroll
    for (int o = 16; o >= 1; o >>= 1) best = min(best, __shfl_xor_sync(0xffffffffu, best, o));
    if (lane == 0) s_best[wic] = best;
    __syncthreads();
    if (threadIdx.x == 0) {
      for (int w = 1; w < (int)(blockDim.x >> 5); ++w) best = min(best, s_best[w]);
      if (best != ~0ull) {
        const int tok = (int)(unsigned)(best & 0xffffffffull) - 1;
        hotidx[tok] = (int8_t)h;
        hotidx[V + tok] = (int8_t)(HOT_TOKENS + h);
        hot_rows[h] = tok;
        hot_rows[HOT_TOKENS + h] = V + tok;
      }
      s_last = best;
    }
    __syncthreads();
    if (s_last == ~0ull) break;
    ++n;
  }
  // fewer tokens than HOT_TOKENS: the unused hot-row numbers point at rows whose counters nobody bumps
  if (threadIdx.x == 0) *picked = n;
}
__global__ void k_inverse_counts(const unsigned long long* __restrict__ counts, int V, int saturate, float* __restrict__ f) {
  for (int v = blockIdx.x * blockDim.x + threadIdx.x; v < V; v += gridDim.x * blockDim.x) {
    unsigned long long c = counts[v];
    if (saturate && c > (1ull << 24)) c = 1ull << 24;  // a float counter stops growing here (model_arrays.cu:413-416)
    f[v] = c ? (float)(1.0 / (double)c) : 0.f;
  }
}

// ---------------------------------------------------------------------------
// NCCL, bound at run time so that a single-GPU process never needs it.
// ---------------------------------------------------------------------------
struct Id128 {
  char bytes[128];
};
struct NcclApi {
  void* lib = nullptr;
  int (*GetUniqueId)(Id128*) = nullptr;
  int (*CommInitRank)(void**, int, Id128, int) = nullptr;  // the id travels by value
  int (*CommDestroy)(void*) = nullptr;
  int (*AllGather)(const void*, void*, size_t, int, void*, cudaStream_t) = nullptr;
  const char* (*GetErrorString)(int) = nullptr;
};
NcclApi g_nccl;

int load_nccl() {
  if (g_nccl.lib) return FV_OK;
  const char* names[] = {"libnccl.so.2", "libnccl.so"};
  void* lib = nullptr;
  for (const char* n : names) {
    lib = dlopen(n, RTLD_NOW | RTLD_GLOBAL);
    if (lib) break;
  }
  if (!lib) return fv::fail(FV_ERR_COMM, "NCCL not found: %s", dlerror());
  NcclApi api;
  api.lib = lib;
  api.GetUniqueId = reinterpret_cast<decltype(api.GetUniqueId)>(dlsym(lib, "ncclGetUniqueId"));
  api.CommInitRank = reinterpret_cast<decltype(api.CommInitRank)>(dlsym(lib, "ncclCommInitRank"));
  api.CommDestroy = reinterpret_cast<decltype(api.CommDestroy)>(dlsym(lib, "ncclCommDestroy"));
  api.AllGather = reinterpret_cast<decltype(api.AllGather)>(dlsym(lib, "ncclAllGather"));
  api.GetErrorString = reinterpret_cast<decltype(api.GetErrorString)>(dlsym(lib, "ncclGetErrorString"));
  if (!api.GetUniqueId || !api.CommInitRank || !api.CommDestroy || !api.AllGather || !api.GetErrorString)
    return fv::fail(FV_ERR_COMM, "NCCL library lacks a required symbol");
  g_nccl = api;
  return FV_OK;
}
constexpr int NCCL_UINT32 = 3;  // ncclUint32 in ncclDataType_t

}  // namespace


// ---------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------
struct fv_trainer {
  fv_config cfg;
  Dev d;
  int device = 0;
  int num_sms = 0;
  int NT = 0;
  cudaStream_t stream = nullptr;
  cudaStream_t copy_stream = nullptr;
  cudaEvent_t ev_begin = nullptr, ev_end = nullptr;
  cudaEvent_t ev_copy[2] = {nullptr, nullptr}, ev_used[2] = {nullptr, nullptr};
  bool have_corpus = false, have_weights = false;
  void* comm = nullptr;
  // owned device buffers
  float* d_wt = nullptr;
  double* d_alpha = nullptr;
  int32_t* d_tokens = nullptr;
  unsigned long long* d_wstart = nullptr;
  unsigned long long* d_perm = nullptr;
  float* d_f = nullptr;
  int32_t* d_idx_stage[2] = {nullptr, nullptr};
  int32_t* d_idx_local[2] = {nullptr, nullptr};  // this rank's ids of a chunk before the all-gather (rank-local host feed)
  uint32_t* d_mail = nullptr;               // local mailbox (flags + packets)
  size_t mail_words = 0;
  uint32_t* peer_mail[16] = {nullptr};      // peers' mailboxes mapped into this process
  uint32_t** d_peer_table = nullptr;
  int comm_mode = 0;                         // 0 none, 1 NCCL all-gather per step, 2 peer-memory mailboxes
  bool linked = false;                       // peers are trainers of this process (fv_trainers_link), not IPC mappings
  bool lockstep = false;                     // linked ranks sharing one device and one stream: phases run rank after rank
  bool own_stream = true;                    // false: `stream` belongs to rank 0 of the group
  unsigned long long* d_xx_acc = nullptr;  // xx_hi [Kp], xx_lo [Kp]
  uint32_t* d_xx_wins = nullptr;
  int32_t* d_cnt = nullptr;
  int32_t* d_cntn = nullptr;
  uint4* d_rec = nullptr;
  int8_t* d_hotidx = nullptr;
  int32_t* d_hot_rows = nullptr;
  uint32_t* d_hot_cnt = nullptr;
  uint32_t* d_hot_cntn = nullptr;
  int hot_rows_picked = 0;       // hot rows the corpus provided (<= HOT_ROWS)
  bool hot_pairs = true;         // option "hot_pairs"
  int tag_forced = 0;            // the "tag_variant" option as given (0: by size)
  bool tag_dedupe_now = false;   // the running call tags with the shared-memory dedupe kernel
  int tag_hot_grid = 0;
  uint32_t* d_colmax = nullptr;
  uint32_t* d_ncb = nullptr;
  double* d_stat_x = nullptr;
  int32_t* d_stat_n = nullptr;
  StepCtl* d_ctl = nullptr;
  float* d_log = nullptr;
  size_t log_cap = 0;
  unsigned long long steps_since_fold = 0;
  unsigned long long ticks = 0;  // host copy of StepCtl::tick
  float delta_now = 0.f;         // anti-Hebbian strength used by the next run_* call
  int tag_un = 1;
  unsigned long long matrix_scans = 0;    // steps in which the column maxima came from a pass over the matrix
  unsigned long long column_rescans = 0;  // single units whose column was read because their candidates were all touched
  bool fused_update = true;      // ordinary steps run evaluation and apply as one kernel (k_update)
  bool fused_this_step = false;
  bool no_grid_meeting = false;  // the running call has collectives of another library in flight beside the step loop
  int update_grid = 0;           // CTAs of k_update: all resident at once
  size_t update_smem = 0;
  unsigned long long update_launches = 0;
  bool cand_dirty = true;  // the candidate lists of the column maxima do not describe the current weights
  int32_t* d_cand_rows = nullptr;
  int32_t* d_cand_n = nullptr;
  uint32_t* d_cand_floor = nullptr;
  uint32_t* d_cand_unc = nullptr;
  unsigned long long* d_colarg = nullptr;
  int tag_batch_u = 1, tag_batch_grid = 0;  // slots per thread and CTAs of the tagging kernel
  int fwd_grid = 0, tag_grid = 0, scan_grid = 0, apply_grid = 0, entry_grid = 0;
  size_t fwd_smem = 0, scan_smem = 0, apply_smem = 0;
};

namespace {

constexpr unsigned long long FOLD_EVERY = 128;  // steps between folds of alpha into wt
constexpr int STAGE_STEPS = 32;                // steps per upload chunk in streaming mode

#define FV_TRY(expr)                    \
  do {                                  \
    int fv_rc_ = (expr);                \
    if (fv_rc_ != FV_OK) return fv_rc_; \
  } while (0)

template <typename T>
int dev_alloc(T** p, size_t count) {
  *p = nullptr;
  FV_CUDA(cudaMalloc(reinterpret_cast<void**>(p), (count ? count : 1) * sizeof(T)));
  return FV_OK;
}

int grid_for(size_t work, int block, int cap) {
  size_t g = (work + block - 1) / block;
  if (g < 1) g = 1;
  if (g > (size_t)cap) g = cap;
  return (int)g;
}

// Launch with programmatic stream serialization (see grid_dependency_wait).
template <typename... KArgs, typename... Args>
cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

template <int NT>
void launch_forward(fv_trainer* tr, int local, const int32_t* idx) {
  launch_pdl(k_forward<NT>, tr->fwd_grid, FWD_THREADS, tr->fwd_smem, tr->stream, tr->d, local, idx);
}
template <int NT>
void forward_occupancy(int* fwd, size_t fwd_smem, cudaError_t* err) {
  *err = cudaOccupancyMaxActiveBlocksPerMultiprocessor(fwd, k_forward<NT>, FWD_THREADS, fwd_smem);
}

#define FV_DISPATCH_NT(nt, fn, ...)     \
  switch (nt) {                         \
    case 1: fn<1>(__VA_ARGS__); break;  \
    case 2: fn<2>(__VA_ARGS__); break;  \
    case 3: fn<3>(__VA_ARGS__); break;  \
    case 4: fn<4>(__VA_ARGS__); break;  \
    case 5: fn<5>(__VA_ARGS__); break;  \
    case 6: fn<6>(__VA_ARGS__); break;  \
    case 7: fn<7>(__VA_ARGS__); break;  \
    default: fn<8>(__VA_ARGS__); break; \
  }

// Multiplies alpha into wt and resets alpha.  `local` = steps already launched
// since the running call began (tr->d.tick0).
int fold_weights(fv_trainer* tr, int local) {
  if (tr->steps_since_fold == 0) return FV_OK;
  k_fold<<<tr->num_sms * 4, 256, 0, tr->stream>>>(tr->d, local);
  k_reset_alpha<<<4, 256, 0, tr->stream>>>(tr->d);
  FV_CUDA(cudaGetLastError());
  tr->steps_since_fold = 0;
  tr->cand_dirty = true;  // every weight changed: the candidate lists are rebuilt in the next step
  return FV_OK;
}

// One global step on tr->stream is five phases, each a kernel (or a short run of kernels):
//   0  forward pass (with NCCL exchange: + k_xx + the all-gather; with emulated ranks: every rank's block in turn)
//   1  exchange kernel (only where several ranks share one stream; otherwise part of phase 2)
//   2  tagging (+ xx_finish and the winner push in its first CTAs)
//   3  evaluation of the normaliser (k_update does this and phase 4 in one launch)
//   4  apply
// `idx` holds this step's input ids (all ranks' windows).  Adds the kernels launched to *launches.
constexpr int STEP_PHASES = 5;
int enqueue_phase(fv_trainer* tr, int phase, int local, const int32_t* idx, uint64_t* launches) {
  const Dev& d = tr->d;
  const bool emulate = (d.flags & FV_FLAG_EMULATE_RANKS) != 0;
  const bool single = (d.G == 1);
  // several ranks on one stream: a rank's winners and xx must be out before any rank tags, so they
  // leave in a kernel of their own (phase 1) instead of in the first CTAs of the tagging kernel
  const bool split_exchange = tr->lockstep && tr->comm_mode == 2 && !emulate && !single;
  if (phase == 1) {
    if (split_exchange) {
      launch_pdl(k_xx, 1 + PUSH_CTAS + (d.hot_x ? HOT_PUSH_CTAS : 0), XX_THREADS, (size_t)0, tr->stream, d, local);
      *launches += 1;
    }
    return FV_OK;
  }
  if (phase > 1) --phase;
  if (phase == 0) {
    if (emulate && !single) {
      // every rank's block in turn, each into its own packet slot
      const int own_rank = tr->d.rank;
      for (int r = 0; r < d.G; ++r) {
        tr->d.rank = r;
        FV_DISPATCH_NT(tr->NT, launch_forward, tr, local, idx);
        launch_pdl(k_xx, 1, XX_THREADS, (size_t)0, tr->stream, tr->d, local);
        *launches += 2;
      }
      tr->d.rank = own_rank;
    } else {
      FV_DISPATCH_NT(tr->NT, launch_forward, tr, local, idx);
      *launches += 1;
      if (tr->comm_mode == 1) {
        // k_xx finishes the packet, one all-gather delivers everybody's
        launch_pdl(k_xx, 1, XX_THREADS, (size_t)0, tr->stream, d, local);
        *launches += 1;
        const int parity = (int)((tr->ticks + (unsigned long long)local) & 1);
        uint32_t* base = tr->d_mail + MAIL_HDR + (size_t)parity * d.G * d.P * 2;  // packets are P 64-bit words
        const int rc = g_nccl.AllGather(base + (size_t)d.rank * d.P * 2, base, (size_t)d.P * 2, NCCL_UINT32, tr->comm, tr->stream);
        if (rc != 0) return fv::fail(FV_ERR_COMM, "ncclAllGather failed: %s", g_nccl.GetErrorString(rc));
      }
    }
  } else if (phase == 1) {
    // One rank, or peer mailboxes: the first CTAs of the tagging kernel compute xx beside the tagging
    // (and, with mailboxes, push winners first and xx last); otherwise xx is complete already.
    const bool fused = single || (tr->comm_mode == 2 && !emulate && !split_exchange);
    const size_t table_smem = tag_table_bytes(tr->tag_un);
    const int xx_ctas = fused ? 1 : 0, push_ctas = (fused && !single) ? PUSH_CTAS + (d.hot_x ? HOT_PUSH_CTAS : 0) : 0;
    // 1: one slot per thread (a step fits one round of the resident threads); 2: dedupe in shared memory;
    // 3: U slots per thread with batched claims (what large steps use)
    const int own = d.shard ? 1 : 0;
    const int u = tr->tag_batch_u;
    const int grid = tr->tag_batch_grid + xx_ctas + push_ctas;
    if (tr->tag_dedupe_now && !own) {
      launch_pdl(k_tag<2>, tr->tag_grid + xx_ctas + push_ctas, XX_THREADS, table_smem, tr->stream, d, local, idx, xx_ctas, push_ctas);
    } else if (u == 1) {
      launch_pdl(k_tag<1>, (d.nhot ? tr->tag_hot_grid + xx_ctas + push_ctas : grid), XX_THREADS, (size_t)0, tr->stream, d, local, idx, xx_ctas, push_ctas);
    } else {
#define FV_TAG_BATCH(U_)                                                                                                      \
  (own ? launch_pdl(k_tag_batch<U_, true>, grid, XX_THREADS, (size_t)0, tr->stream, d, local, idx, xx_ctas, push_ctas)   \
       : launch_pdl(k_tag_batch<U_, false>, grid, XX_THREADS, (size_t)0, tr->stream, d, local, idx, xx_ctas, push_ctas))
      if (u == 2) FV_TAG_BATCH(2);
      else if (u == 4) FV_TAG_BATCH(4);
      else FV_TAG_BATCH(8);
#undef FV_TAG_BATCH
    }
    *launches += 1;
  } else if (phase == 2) {
    tr->fused_this_step = false;
    if (d.use_cand && !tr->cand_dirty && !d.shard && tr->fused_update && tr->update_grid > 0 && !tr->no_grid_meeting) {
      // an ordinary step: evaluation and apply in one kernel
      const int qblocks = (d.K + SCAN_THREADS / 32 - 1) / (SCAN_THREADS / 32);
      tr->update_launches += 1;
      launch_pdl(k_update, tr->update_grid, SCAN_THREADS, tr->update_smem, tr->stream, d, local, idx, qblocks,
                 tr->update_launches * (unsigned long long)tr->update_grid);
      FV_CUDA(cudaGetLastError());
      *launches += 1;
      tr->fused_this_step = true;
      tr->steps_since_fold += 1;
    } else if (d.use_cand) {
      const int rebuild = tr->cand_dirty ? 1 : 0;
      const int qblocks = (d.K + SCAN_THREADS / 32 - 1) / (SCAN_THREADS / 32);  // a warp per unit
      const int rblocks = std::max(tr->scan_grid - qblocks, tr->num_sms);  // one resident wave together with the query CTAs
      launch_pdl(k_eval, rblocks + qblocks, SCAN_THREADS, tr->scan_smem, tr->stream, d, local, idx, rebuild, qblocks);
      *launches += 1;
      if (rebuild) {
        launch_pdl(k_colscan, tr->scan_grid, SCAN_THREADS, (size_t)d.Kp * sizeof(unsigned long long), tr->stream, d, local, rebuild);
        launch_pdl(k_collect, tr->scan_grid, SCAN_THREADS, (size_t)0, tr->stream, d);
        *launches += 2;
        tr->cand_dirty = false;
        tr->matrix_scans += 1;
      }
    } else {
      launch_pdl(k_scan, tr->scan_grid, SCAN_THREADS, tr->scan_smem, tr->stream, d, local, idx);
      *launches += 1;
    }
  } else if (!tr->fused_this_step) {
    launch_pdl(k_apply, tr->apply_grid, 256, tr->apply_smem, tr->stream, d, local, idx);
    FV_CUDA(cudaGetLastError());
    *launches += 1;
    tr->steps_since_fold += 1;
  }
  return FV_OK;
}

int ensure_log(fv_trainer* tr, size_t nsteps) {
  if (tr->log_cap >= nsteps) return FV_OK;
  if (tr->d_log) FV_CUDA(cudaFree(tr->d_log));
  tr->d_log = nullptr;
  tr->log_cap = 0;
  FV_TRY(dev_alloc(&tr->d_log, 2 * nsteps));
  tr->log_cap = nsteps;
  tr->d.nc_log = tr->d_log;
  tr->d.s_log = tr->d_log + nsteps;
  return FV_OK;
}

// The step loop of one rank, cut into pieces so that several ranks driven by one host thread can be
// advanced phase by phase (see run_group_lockstep).  idx_host == nullptr: ids are built on the GPU from
// the corpus and the current order.  Otherwise they are uploaded in chunks of STAGE_STEPS steps on a
// second stream, two chunks in flight.  idx_local: idx_host holds only this rank's windows
// (nsteps * batch of them); the ranks' blocks of a chunk are then all-gathered over NVLink on the
// second stream, so every rank uploads 1/world of the ids.
struct StepLoop {
  unsigned long long first_step = 0, nsteps = 0, timed_from = 0;
  float eps = 0.f;
  const int32_t* idx_host = nullptr;
  bool idx_local = false, gather_ids = false;
  size_t step_ids = 0, own_ids = 0;
  unsigned long long chunk_id = 0, fold_every = FOLD_EVERY;
  int chunk_rstride = 0;
  const int32_t* idx = nullptr;  // ids of the step being enqueued
  uint64_t launches = 0;
};

int loop_begin(fv_trainer* tr, StepLoop& L) {
  FV_REQUIRE(tr->have_weights, FV_ERR_STATE, "trainer has no weights: call fv_trainer_set_weights first");
  if (!L.idx_host) FV_REQUIRE(tr->have_corpus, FV_ERR_STATE, "trainer has no corpus: call fv_trainer_set_corpus first");
  if (tr->d.G > 1 && !(tr->d.flags & FV_FLAG_EMULATE_RANKS))
    FV_REQUIRE(tr->comm_mode != 0, FV_ERR_STATE, "world > 1 but neither fv_trainer_init_comm nor fv_trainers_link was called");
  FV_REQUIRE(L.nsteps >= 1 && L.nsteps <= (1ull << 30), FV_ERR_INVALID, "number of steps must be in [1, 2^30]");
  FV_REQUIRE(L.timed_from < L.nsteps, FV_ERR_INVALID, "timed_from must be smaller than the number of steps");
  FV_TRY(ensure_log(tr, L.nsteps));
  const Dev& d = tr->d;
  L.fold_every = (d.flags & FV_FLAG_FOLD_EVERY_STEP) ? 1 : FOLD_EVERY;
  L.step_ids = (size_t)d.G * d.B * d.W;
  L.own_ids = (size_t)d.B * d.W;
  for (int b = 0; b < 2; ++b)
    if (!tr->d_idx_stage[b]) FV_TRY(dev_alloc(&tr->d_idx_stage[b], L.step_ids * STAGE_STEPS));
  L.gather_ids = L.idx_host && L.idx_local && d.G > 1 && !(d.flags & FV_FLAG_EMULATE_RANKS);
  // The ranks' ids meet through NCCL all-gathers on the second stream while the step loop runs.  A kernel whose own
  // CTAs wait for one another (k_update's meeting point) needs its whole grid resident; beside an NCCL kernel it
  // may not get that until the collective ends, and the collective may be waiting for a rank whose GPU is filled
  // by a tagging kernel that waits for this rank's next packet: the ring closes (seen on 8 GPUs as FV_ERR_TIMEOUT
  // at the first block boundary).  Such calls evaluate and apply in two kernels, which wait for nobody on the
  // same GPU.
  tr->no_grid_meeting = L.gather_ids;
  if (L.idx_host && L.idx_local && d.G > 1 && !L.gather_ids)
    return fv::fail(FV_ERR_INVALID, "rank-local ids need real ranks: with FV_FLAG_EMULATE_RANKS pass all ranks' ids");
  if (L.gather_ids) FV_REQUIRE(tr->comm != nullptr, FV_ERR_STATE, "rank-local ids travel through the NCCL communicator: call fv_trainer_init_comm");
  for (int b = 0; b < 2 && L.gather_ids; ++b)
    if (!tr->d_idx_local[b]) FV_TRY(dev_alloc(&tr->d_idx_local[b], L.own_ids * STAGE_STEPS));
  tr->d.idx_rstride = (int)L.own_ids;
  tr->d.tick0 = tr->ticks;
  {
    // Hot pairs: with one rank, emulated ranks, or ranks that exchange their counts through peer mailboxes every
    // hot-row slot is counted by some forward pass, and large steps need no dedupe any more (several slots per
    // thread, batched claims).  Ranks that cannot exchange the counts (NCCL mode) count their own windows only;
    // their large steps keep the dedupe kernel, which does not claim hot pairs.
    Dev& dd = tr->d;
    const bool emu = (dd.flags & FV_FLAG_EMULATE_RANKS) != 0;
    const bool can_x = dd.G > 1 && !emu && tr->comm_mode == 2;
    const bool all_counted = dd.G == 1 || emu || can_x;
    const bool want_hot = tr->hot_pairs && !dd.shard && tr->hot_rows_picked > 0;
    const bool big = tr->tag_un == 2;  // a step larger than one round of k_tag<1>
    tr->tag_dedupe_now = big && !dd.shard && (tr->tag_forced == 2 || !(want_hot && all_counted));
    dd.nhot = (want_hot && !tr->tag_dedupe_now) ? tr->hot_rows_picked : 0;
    dd.hot_x = (dd.nhot && can_x) ? 1 : 0;
  }
  L.chunk_rstride = (int)L.own_ids;
  k_set_ctl<<<1, 1, 0, tr->stream>>>(tr->d_ctl, L.first_step, L.eps, tr->delta_now);
  L.launches = 1;
  return FV_OK;
}

// Before step k: the timing mark, and at the start of a chunk the ids of its steps.
int loop_stage(fv_trainer* tr, StepLoop& L, unsigned long long k) {
  const Dev& d = tr->d;
  if (k == L.timed_from) {
    // the timed region starts here: steps before it are warm-up inside the same call
    if (k > 0) {
      k_reset_phase_clock<<<1, 1, 0, tr->stream>>>(tr->d_ctl);
      L.launches += 1;
    }
    FV_CUDA(cudaEventRecord(tr->ev_begin, tr->stream));
  }
  // Input ids arrive in chunks of STAGE_STEPS steps through two device buffers filled on a second
  // stream, one chunk ahead of the step loop: uploaded from the caller's host memory, or derived
  // from the resident corpus and window order.
  const int b = (int)(L.chunk_id & 1);
  if (k % STAGE_STEPS == 0) {
    const unsigned long long n = (L.nsteps - k < STAGE_STEPS) ? L.nsteps - k : STAGE_STEPS;
    // the buffer must no longer be read by the chunk that used it two chunks ago
    if (L.chunk_id >= 2) FV_CUDA(cudaStreamWaitEvent(tr->copy_stream, tr->ev_used[b], 0));
    if (L.gather_ids) {
      // this rank's ids of the chunk go up, then one all-gather lays the ranks' blocks side by side:
      // [rank][step of the chunk][B*w], i.e. the blocks of one step lie n * B*w apart
      FV_CUDA(cudaMemcpyAsync(tr->d_idx_local[b], L.idx_host + k * L.own_ids, n * L.own_ids * sizeof(int32_t),
                              cudaMemcpyHostToDevice, tr->copy_stream));
      // comm mode 1 already uses the communicator on the step stream: keep NCCL calls in one order there
      cudaStream_t gs = (tr->comm_mode == 1) ? tr->stream : tr->copy_stream;
      if (gs != tr->copy_stream) {
        FV_CUDA(cudaEventRecord(tr->ev_copy[b], tr->copy_stream));
        FV_CUDA(cudaStreamWaitEvent(gs, tr->ev_copy[b], 0));
      }
      const int rc = g_nccl.AllGather(tr->d_idx_local[b], tr->d_idx_stage[b], n * L.own_ids, NCCL_UINT32, tr->comm, gs);
      if (rc != 0) return fv::fail(FV_ERR_COMM, "ncclAllGather (ids) failed: %s", g_nccl.GetErrorString(rc));
      L.chunk_rstride = (int)(n * L.own_ids);
    } else if (L.idx_host) {
      L.chunk_rstride = (int)L.own_ids;
      FV_CUDA(cudaMemcpyAsync(tr->d_idx_stage[b], L.idx_host + k * L.step_ids, n * L.step_ids * sizeof(int32_t),
                              cudaMemcpyHostToDevice, tr->copy_stream));
    } else {
      k_build_idx_block<<<tr->num_sms * 4, 256, 0, tr->copy_stream>>>(d, L.first_step + k, (int)n, tr->d_idx_stage[b]);
      L.launches += 1;
    }
    FV_CUDA(cudaEventRecord(tr->ev_copy[b], tr->copy_stream));
    FV_CUDA(cudaStreamWaitEvent(tr->stream, tr->ev_copy[b], 0));
    if (L.idx_host) {
      k_check_idx<<<tr->entry_grid, 256, 0, tr->stream>>>(d, tr->d_idx_stage[b], n * L.step_ids);
      L.launches += 1;
    }
  }
  tr->d.idx_rstride = L.chunk_rstride;
  L.idx = tr->d_idx_stage[b] + (k % STAGE_STEPS) * (L.gather_ids ? L.own_ids : L.step_ids);
  return FV_OK;
}

int loop_after_step(fv_trainer* tr, StepLoop& L, unsigned long long k) {
  if ((k + 1) % STAGE_STEPS == 0 || k + 1 == L.nsteps) {
    FV_CUDA(cudaEventRecord(tr->ev_used[L.chunk_id & 1], tr->stream));
    ++L.chunk_id;
  }
  if (tr->steps_since_fold >= L.fold_every) {
    FV_TRY(fold_weights(tr, (int)(k + 1)));
    L.launches += 2;
  }
  return FV_OK;
}

int loop_end(fv_trainer* tr, StepLoop& L, float* nc_out, float* scale_out, fv_run_stats* stats) {
  const Dev& d = tr->d;
  const unsigned long long nsteps = L.nsteps;
  tr->d.idx_rstride = (int)L.own_ids;
  k_advance<<<1, 1, 0, tr->stream>>>(tr->d_ctl, nsteps);
  tr->ticks += nsteps;
  L.launches += 1;
  FV_CUDA(cudaEventRecord(tr->ev_end, tr->stream));
  std::vector<float> log(2 * nsteps);
  FV_CUDA(cudaMemcpyAsync(log.data(), tr->d.nc_log, nsteps * sizeof(float), cudaMemcpyDeviceToHost, tr->stream));
  FV_CUDA(cudaMemcpyAsync(log.data() + nsteps, tr->d.s_log, nsteps * sizeof(float), cudaMemcpyDeviceToHost,
                          tr->stream));
  FV_CUDA(cudaStreamSynchronize(tr->stream));
  if (nc_out) memcpy(nc_out, log.data(), nsteps * sizeof(float));
  if (scale_out) memcpy(scale_out, log.data() + nsteps, nsteps * sizeof(float));

  StepCtl h;
  FV_CUDA(cudaMemcpy(&h, tr->d_ctl, sizeof(h), cudaMemcpyDeviceToHost));
  const uint32_t dev_err = h.error;
  if (!tr->d.use_cand) tr->matrix_scans += nsteps;
  tr->column_rescans += h.scans_run;
  const unsigned long long timed = nsteps - L.timed_from;
  if (getenv("FV_STAMPS")) {
    fprintf(stderr, "[rank %d] per step (us): other %.1f forward %.1f xx %.1f wait %.1f tag %.1f scan %.1f apply %.1f fold %.1f\n", tr->d.rank,
            h.phase_ns[PH_OTHER] * 1e-3 / timed, h.phase_ns[PH_FORWARD] * 1e-3 / timed, h.phase_ns[PH_XX] * 1e-3 / timed,
            h.phase_ns[PH_WAIT] * 1e-3 / timed, h.phase_ns[PH_TAG] * 1e-3 / timed, h.phase_ns[PH_SCAN] * 1e-3 / timed,
            h.phase_ns[PH_APPLY] * 1e-3 / timed, h.phase_ns[PH_FOLD] * 1e-3 / timed);
  }
  if (stats) {
    memset(stats, 0, sizeof(*stats));
    float ms = 0.f;
    FV_CUDA(cudaEventElapsedTime(&ms, tr->ev_begin, tr->ev_end));
    stats->steps = nsteps;
    unsigned long long mine = 0;
    for (unsigned long long k = L.timed_from; k < nsteps; ++k) {
      if (L.idx_host) {
        mine += d.B;
      } else {
        uint64_t first, cnt;
        fv_shard_range(d.Ns, d.B, d.G, d.rank, L.first_step + k, &first, &cnt);
        mine += cnt;
      }
    }
    stats->windows = mine;
    stats->seconds = ms * 1e-3;
    // from the device-side phase clock (the timed steps, no sampling): forward; xx + waiting for the peers;
    // tag + scan + apply.  Folding and the gaps between steps make up the rest of `seconds`.
    stats->fwd_seconds = h.phase_ns[PH_FORWARD] * 1e-9;
    stats->exch_seconds = (h.phase_ns[PH_XX] + h.phase_ns[PH_WAIT]) * 1e-9;
    stats->upd_seconds = (h.phase_ns[PH_TAG] + h.phase_ns[PH_SCAN] + h.phase_ns[PH_APPLY]) * 1e-9;
    stats->kernel_launches = L.launches;
    stats->last_nc = log[nsteps - 1];
    stats->last_scale = log[2 * nsteps - 1];
    stats->device_error = dev_err;
    stats->timed_steps = (uint32_t)timed;
  }
  if (dev_err & FV_DEVERR_TOKEN_RANGE) return fv::fail(FV_ERR_DATA, "a token id was outside [0, V) (device check)");
  if (dev_err & FV_DEVERR_WINDOW_RANGE)
    return fv::fail(FV_ERR_DATA, "a window order entry or window start was out of range (device check)");
  if (dev_err & FV_DEVERR_TIMEOUT)
    return fv::fail(FV_ERR_TIMEOUT, "a peer rank did not deliver its step packet in time; the replicas are out of step");
  if (dev_err & FV_DEVERR_NAN_WEIGHT)
    return fv::fail(FV_ERR_DATA, "a weight was NaN or a unit's scale collapsed to zero (device check)");
  if (dev_err & FV_DEVERR_SLOT_RANGE)
    return fv::fail(FV_ERR_DATA, "a scatter record or a peer's update entry was out of range (device check)");
  return FV_OK;
}

int run_steps_impl(fv_trainer* tr, unsigned long long first_step, unsigned long long nsteps, float eps,
                   const int32_t* idx_host, bool idx_local, float* nc_out, float* scale_out, fv_run_stats* stats,
                   unsigned long long timed_from = 0) {
  if (stats) memset(stats, 0, sizeof(*stats));
  if (nsteps == 0) return FV_OK;
  fv::DeviceGuard guard(tr->device);
  FV_REQUIRE(guard.ok, FV_ERR_CUDA, "cannot select device %d", tr->device);
  StepLoop L;
  L.first_step = first_step;
  L.nsteps = nsteps;
  L.eps = eps;
  L.idx_host = idx_host;
  L.idx_local = idx_local;
  L.timed_from = timed_from;
  FV_TRY(loop_begin(tr, L));
  for (unsigned long long k = 0; k < nsteps; ++k) {
    FV_TRY(loop_stage(tr, L, k));
    for (int ph = 0; ph < STEP_PHASES; ++ph) FV_TRY(enqueue_phase(tr, ph, (int)k, L.idx, &L.launches));
    FV_TRY(loop_after_step(tr, L, k));
  }
  return loop_end(tr, L, nc_out, scale_out, stats);
}

void free_all(fv_trainer* tr) {
  cudaSetDevice(tr->device);
  for (int r = 0; r < 16 && !tr->linked; ++r)
    if (tr->peer_mail[r] && r != tr->d.rank) cudaIpcCloseMemHandle(tr->peer_mail[r]);
  if (tr->comm && g_nccl.CommDestroy) g_nccl.CommDestroy(tr->comm);
  void* bufs[] = {tr->d_wt,  tr->d_alpha, tr->d_tokens, tr->d_wstart, tr->d_perm,   tr->d_f,
                  tr->d_mail, tr->d_peer_table, tr->d_xx_acc, tr->d_xx_wins, tr->d_cnt, tr->d_cntn, tr->d_rec, tr->d_hotidx, tr->d_hot_rows, tr->d_hot_cnt, tr->d_hot_cntn, tr->d_colmax, tr->d_ncb, tr->d_stat_x, tr->d_stat_n, tr->d_cand_rows, tr->d_cand_n, tr->d_cand_floor, tr->d_cand_unc, tr->d_colarg, tr->d_ctl,
                  tr->d_log, tr->d_idx_stage[0], tr->d_idx_stage[1], tr->d_idx_local[0], tr->d_idx_local[1]};
  for (void* b : bufs)
    if (b) cudaFree(b);
  cudaEvent_t evs[] = {tr->ev_begin, tr->ev_end, tr->ev_copy[0], tr->ev_copy[1], tr->ev_used[0], tr->ev_used[1]};
  for (cudaEvent_t e : evs)
    if (e) cudaEventDestroy(e);
  if (tr->stream && tr->own_stream) cudaStreamDestroy(tr->stream);
  if (tr->copy_stream) cudaStreamDestroy(tr->copy_stream);
  delete tr;
}

// Sharded or replicated update once the ranks can write into one another's mailboxes (the "shard" option
// and the environment variable FV_SHARD = 0 / 1 choose; the anti-Hebbian term needs the replicated one).
int default_shard(const fv_trainer* tr) {
  if (tr->d.has_delta || tr->d.G < 2) return 0;
  const char* e = getenv("FV_SHARD");
  if (e) return atoi(e) != 0;
  // Measured on 2 and 4 B200s (config 1 shapes) the replicated update is the faster one: 57.7 against 62.9 us
  // and 67.2 against 75.8 us per global step -- the second exchange of the sharded update (counts and partial
  // normalisers) costs more than the bookkeeping it saves at these sizes.
  return 0;
}

// Which tagging kernel runs and on how many CTAs.  force_un = 0: by the size of a step.
void choose_tag_variant(fv_trainer* tr, int force_un) {
  const Dev& d = tr->d;
  const size_t E = (size_t)d.G * d.B * d.W * (1 + d.has_delta);
  const size_t resident = (size_t)tr->num_sms * 3 - 1 - PUSH_CTAS - HOT_PUSH_CTAS;
  // tag_un = 2: the step is larger than one round of the one-slot-per-thread kernel.  Such a step takes several
  // slots per thread with batched claims when every hot-row slot is counted (see loop_begin), else it deduplicates
  // in shared memory: measured at 8 ranks' slots with every request claiming for itself, 46.6 us for the three
  // update kernels with the dedupe against 55.4 us with four batched slots per thread -- hot (unit, token) pairs
  // meet at one L2 address -- and 29 us with the batched kernel once the hot pairs are counted
  tr->tag_un = (force_un == 2 || (force_un == 0 && (E + XX_THREADS - 1) / XX_THREADS > resident)) ? 2 : 1;
  tr->tag_grid = grid_for(E, XX_THREADS * tr->tag_un, (int)resident);
  // slots per thread so that one block round covers the step
  int u = 1;
  while (u < 8 && (E + (size_t)XX_THREADS * u - 1) / ((size_t)XX_THREADS * u) > resident) u *= 2;
  if (force_un == 1) u = 1;
  tr->tag_batch_u = u;
  tr->tag_batch_grid = grid_for(E, XX_THREADS * u, (int)resident);
  // hot pairs ride behind the slots of the one-slot-per-thread kernel; where the slots alone fill the resident
  // threads (two ranks of 10000 windows), a tenth of the CTAs takes a second block round for them
  const size_t with_hot = E + (size_t)HOT_ROWS * d.Kp;
  tr->tag_forced = force_un;
  tr->tag_hot_grid = grid_for(with_hot, XX_THREADS, (int)resident);
}

int create_impl(const fv_config* cfg, fv_trainer* tr) {
  tr->cfg = *cfg;
  tr->device = cfg->device;
  tr->delta_now = cfg->delta;
  FV_CUDA(cudaSetDevice(cfg->device));
  cudaDeviceProp prop;
  FV_CUDA(cudaGetDeviceProperties(&prop, cfg->device));
  tr->num_sms = prop.multiProcessorCount;
  FV_CUDA(cudaStreamCreateWithFlags(&tr->stream, cudaStreamNonBlocking));
  FV_CUDA(cudaStreamCreateWithFlags(&tr->copy_stream, cudaStreamNonBlocking));
  FV_CUDA(cudaEventCreate(&tr->ev_begin));
  FV_CUDA(cudaEventCreate(&tr->ev_end));
  for (int b = 0; b < 2; ++b) {
    FV_CUDA(cudaEventCreateWithFlags(&tr->ev_copy[b], cudaEventDisableTiming));
    FV_CUDA(cudaEventCreateWithFlags(&tr->ev_used[b], cudaEventDisableTiming));
  }

  Dev& d = tr->d;
  memset(&d, 0, sizeof(d));
  d.K = (int)cfg->hid;
  d.Kp = (d.K + 3) & ~3;
  d.Kq = d.Kp / 4;
  d.V = (int)cfg->vocab;
  d.N = 2 * d.V;
  d.W = (int)cfg->window;
  d.B = (int)cfg->batch;
  d.G = cfg->world;
  d.rank = cfg->rank;
  d.has_delta = (cfg->delta != 0.0f) ? 1 : 0;
  d.MO = (d.B + 3) & ~3;                  // second winners (with delta) start here (64-bit words)
  d.XO = d.MO * (1 + d.has_delta);        // xx follows
  d.P = d.XO + d.Kp;
  d.idx_rstride = d.B * d.W;
  d.spin_limit = 8u << 20;  // ~10 s of polling with back-off
  {
    auto magic = [](uint32_t divisor, uint32_t* m, uint32_t* s) {
      uint32_t l = 0;
      while ((1ull << l) < divisor) ++l;
      *s = 31 + l;
      *m = (uint32_t)(((1ull << *s) + divisor - 1) / divisor);
    };
    magic((uint32_t)d.W, &d.mW, &d.sW);
    magic((uint32_t)d.B, &d.mB, &d.sB);
    magic((uint32_t)d.Kp, &d.mKp, &d.sKp);
    magic((uint32_t)d.G, &d.mG, &d.sG);
  }
  d.prec = cfg->prec;
  d.flags = cfg->flags;
  tr->NT = (d.Kq + 31) / 32;

  size_t E = (size_t)d.G * d.B * d.W * (1 + (cfg->delta != 0.0f ? 1 : 0));  // virtual slots: both kinds with delta
  FV_TRY(dev_alloc(&tr->d_wt, ((size_t)d.N + 1) * d.Kp));  // one extra all-zero row for padding positions
  FV_TRY(dev_alloc(&tr->d_alpha, 2 * (size_t)d.Kp));
  FV_TRY(dev_alloc(&tr->d_f, (size_t)d.V));
  d.inbox_off = (MAIL_HDR + 2 * 2 * (size_t)d.G * d.P + 3) & ~(size_t)3;
  d.inbox_cap = (d.G > 1 && !d.has_delta) ? (size_t)d.G * d.B * d.W : 0;  // a sender's list can hold every slot of a step
  tr->mail_words = d.inbox_off + 2 * (size_t)d.G * d.inbox_cap;
  d.HC = HOT_ROWS * d.Kp * (1 + d.has_delta);
  d.hot_off = (tr->mail_words + 3) & ~(size_t)3;
  d.hot_x = 0;
  if (d.G > 1) tr->mail_words = d.hot_off + 2 * 2 * (size_t)d.G * d.HC;  // u64 [2][G][HC]
  FV_TRY(dev_alloc(&tr->d_mail, tr->mail_words));
  const size_t hot_pairs = (size_t)HOT_ROWS * d.Kp;
  E += hot_pairs;  // records: one per slot, one per hot pair
  d.rec_cap = (int)E;
  FV_TRY(dev_alloc(&tr->d_cnt, E));
  if (cfg->delta != 0.0f) {
    FV_TRY(dev_alloc(&tr->d_cntn, E));
    FV_CUDA(cudaMemsetAsync(tr->d_cntn, 0, E * sizeof(int32_t), tr->stream));
    FV_TRY(dev_alloc(&tr->d_hot_cntn, hot_pairs));
    FV_CUDA(cudaMemsetAsync(tr->d_hot_cntn, 0, hot_pairs * sizeof(uint32_t), tr->stream));
  }
  FV_TRY(dev_alloc(&tr->d_rec, E));
  FV_TRY(dev_alloc(&tr->d_hotidx, (size_t)d.N + 1));
  FV_TRY(dev_alloc(&tr->d_hot_rows, (size_t)HOT_ROWS));
  FV_TRY(dev_alloc(&tr->d_hot_cnt, hot_pairs));
  FV_CUDA(cudaMemsetAsync(tr->d_hotidx, 0xff, (size_t)d.N + 1, tr->stream));
  FV_CUDA(cudaMemsetAsync(tr->d_hot_rows, 0, HOT_ROWS * sizeof(int32_t), tr->stream));
  FV_CUDA(cudaMemsetAsync(tr->d_hot_cnt, 0, hot_pairs * sizeof(uint32_t), tr->stream));
  d.hotidx = tr->d_hotidx;
  d.hot_rows = tr->d_hot_rows;
  d.hot_cnt = tr->d_hot_cnt;
  d.hot_cntn = tr->d_hot_cntn;
  d.nhot = 0;
  FV_TRY(dev_alloc(&tr->d_colmax, 2 * (size_t)d.Kp));
  FV_TRY(dev_alloc(&tr->d_ncb, 2));
  FV_TRY(dev_alloc(&tr->d_cand_rows, (size_t)d.Kp * CAND_CAP));
  FV_TRY(dev_alloc(&tr->d_cand_n, (size_t)d.Kp));
  FV_TRY(dev_alloc(&tr->d_cand_floor, (size_t)d.Kp));
  FV_TRY(dev_alloc(&tr->d_cand_unc, (size_t)d.Kp));
  FV_TRY(dev_alloc(&tr->d_colarg, (size_t)d.Kp));
  FV_CUDA(cudaMemsetAsync(tr->d_cand_rows, 0, (size_t)d.Kp * CAND_CAP * sizeof(int32_t), tr->stream));
  FV_CUDA(cudaMemsetAsync(tr->d_cand_n, 0, (size_t)d.Kp * sizeof(int32_t), tr->stream));
  FV_CUDA(cudaMemsetAsync(tr->d_cand_floor, 0xff, (size_t)d.Kp * sizeof(uint32_t), tr->stream));
  FV_CUDA(cudaMemsetAsync(tr->d_cand_unc, 0, (size_t)d.Kp * sizeof(uint32_t), tr->stream));
  FV_CUDA(cudaMemsetAsync(tr->d_colarg, 0, (size_t)d.Kp * sizeof(unsigned long long), tr->stream));
  d.cand_rows = tr->d_cand_rows;
  d.cand_n = tr->d_cand_n;
  d.cand_floor = tr->d_cand_floor;
  d.cand_unc = tr->d_cand_unc;
  d.colarg = tr->d_colarg;
  {
    const char* e = getenv("FV_COLMAX");  // "scan": stream the matrix in every step instead of keeping candidate lists
    d.use_cand = (e && strcmp(e, "scan") == 0) ? 0 : 1;
  }
  FV_TRY(dev_alloc(&tr->d_stat_x, 2 * (size_t)d.Kp));
  FV_TRY(dev_alloc(&tr->d_stat_n, 2 * (size_t)d.Kp));
  FV_TRY(dev_alloc(&tr->d_ctl, 1));
  FV_CUDA(cudaMemsetAsync(tr->d_cnt, 0, E * sizeof(int32_t), tr->stream));
  // a record whose last word is zero is a hole; k_apply returns every used record to that state, so the
  // list must start out as all holes (memory recycled from an earlier allocation is not zero)
  FV_CUDA(cudaMemsetAsync(tr->d_rec, 0, E * sizeof(uint4), tr->stream));
  FV_CUDA(cudaMemsetAsync(tr->d_colmax, 0, 2 * (size_t)d.Kp * sizeof(uint32_t), tr->stream));
  FV_CUDA(cudaMemsetAsync(tr->d_ncb, 0, 2 * sizeof(uint32_t), tr->stream));
  FV_CUDA(cudaMemsetAsync(tr->d_ctl, 0, sizeof(StepCtl), tr->stream));
  FV_CUDA(cudaMemsetAsync(tr->d_mail, 0, tr->mail_words * sizeof(uint32_t), tr->stream));
  FV_CUDA(cudaMemsetAsync(tr->d_f, 0, (size_t)d.V * sizeof(float), tr->stream));
  d.wt = tr->d_wt;
  d.alpha = tr->d_alpha;
  d.f = tr->d_f;
  d.mail = tr->d_mail;
  d.peers = nullptr;
  d.cnt = tr->d_cnt;
  d.cntn = tr->d_cntn;
  d.rec = tr->d_rec;
  d.colmax = tr->d_colmax;
  d.ncb = tr->d_ncb;
  d.stat_x = tr->d_stat_x;
  d.stat_n = tr->d_stat_n;
  d.ctl = tr->d_ctl;
  k_reset_alpha<<<4, 256, 0, tr->stream>>>(d);
  FV_CUDA(cudaGetLastError());

  // launch geometry: whole multiples of the SM count
  tr->fwd_smem = (size_t)d.Kp * sizeof(float);
  tr->scan_smem = (size_t)d.Kp * (sizeof(double) + sizeof(int) + 2 * sizeof(uint32_t));
  tr->apply_smem = (size_t)d.Kp * (sizeof(double) + sizeof(int) + sizeof(uint32_t));
  int fwd_bps = 0;
  cudaError_t oerr = cudaSuccess;
  FV_DISPATCH_NT(tr->NT, forward_occupancy, &fwd_bps, tr->fwd_smem, &oerr);
  FV_CUDA(oerr);
  if (fwd_bps < 1) fwd_bps = 1;
  tr->fwd_grid = grid_for((size_t)d.B * 32, FWD_THREADS, tr->num_sms * fwd_bps);
  tr->scan_grid = tr->num_sms * 2;
  // small steps: one slot per thread keeps enough CTAs busy; large steps deduplicate 1024 slots per CTA
  // Three CTAs fit an SM (registers); the grid stays resident together with the 1 + PUSH_CTAS CTAs that
  // serve the exchange.  A CTA takes 512 slots per block round while one round covers the step, else
  // 1024 deduplicated in shared memory (2048 per round measured no faster at 8 ranks).
  {
    const char* e = getenv("FV_TAG_VARIANT");  // same as the "tag_variant" option, for whole runs
    choose_tag_variant(tr, e ? atoi(e) : 0);
  }
  tr->entry_grid = grid_for(E, 256, tr->num_sms * 8);
  {
    // k_apply waits on peers inside the kernel (sharded update), so its grid must be fully resident
    int apply_bps = 0;
    FV_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&apply_bps, k_apply, 256, tr->apply_smem));
    if (apply_bps < 1) apply_bps = 1;
    if (apply_bps > 4) apply_bps = 4;
    tr->apply_grid = grid_for(E, 256, tr->num_sms * apply_bps);
  }
  {
    // k_update's CTAs meet inside the kernel, so the whole grid must be resident
    tr->update_smem = (size_t)d.Kp * (3 * sizeof(double) + sizeof(int) + 2 * sizeof(uint32_t));
    int bps = 0;
    FV_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&bps, k_update, SCAN_THREADS, tr->update_smem));
    if (bps > 2) bps = 2;
    const int qblocks = (d.K + SCAN_THREADS / 32 - 1) / (SCAN_THREADS / 32);
    tr->update_grid = (bps >= 1 && tr->num_sms * bps > qblocks + tr->num_sms / 2) ? tr->num_sms * bps : 0;
    const char* e = getenv("FV_FUSED_UPDATE");
    tr->fused_update = e ? atoi(e) != 0 : true;
    const char* hp = getenv("FV_HOT_PAIRS");
    tr->hot_pairs = hp ? atoi(hp) != 0 : true;
  }
  FV_TRY(dev_alloc(&tr->d_xx_acc, 2 * (size_t)XX_SLOTS * d.Kp));
  FV_TRY(dev_alloc(&tr->d_xx_wins, (size_t)d.Kp));
  FV_CUDA(cudaMemsetAsync(tr->d_xx_acc, 0, 2 * (size_t)XX_SLOTS * d.Kp * sizeof(unsigned long long), tr->stream));
  FV_CUDA(cudaMemsetAsync(tr->d_xx_wins, 0, (size_t)d.Kp * sizeof(uint32_t), tr->stream));
  d.xx_hi = tr->d_xx_acc;
  d.xx_lo = tr->d_xx_acc + (size_t)XX_SLOTS * d.Kp;
  d.xx_wins = tr->d_xx_wins;
  d.fmax = 1.0f;
  FV_CUDA(cudaMemsetAsync(tr->d_wt, 0, ((size_t)d.N + 1) * d.Kp * sizeof(float), tr->stream));
  FV_CUDA(cudaStreamSynchronize(tr->stream));
  return FV_OK;
}

}  // namespace

extern "C" {

int fv_trainer_create(const fv_config* cfg, fv_trainer** out) {
  FV_REQUIRE(cfg && out, FV_ERR_INVALID, "fv_trainer_create: NULL argument");
  *out = nullptr;
  FV_REQUIRE(cfg->struct_size == sizeof(fv_config), FV_ERR_INVALID,
             "fv_trainer_create: struct_size %u != %zu (ABI mismatch)", cfg->struct_size, sizeof(fv_config));
  FV_REQUIRE(cfg->hid >= 1 && cfg->hid <= MAX_K, FV_ERR_INVALID, "hid must be in [1, %d], got %u", MAX_K, cfg->hid);
  FV_REQUIRE(cfg->vocab >= 1 && cfg->vocab <= (1u << 29), FV_ERR_INVALID, "vocab out of range: %u", cfg->vocab);
  FV_REQUIRE(cfg->window >= 1 && cfg->window <= 32, FV_ERR_INVALID, "window must be in [1, 32], got %u", cfg->window);
  FV_REQUIRE(cfg->batch >= 1, FV_ERR_INVALID, "batch must be >= 1");
  FV_REQUIRE((2ull * cfg->vocab + 1) * ((cfg->hid + 3ull) & ~3ull) < (1ull << 31), FV_ERR_INVALID,
             "(2*vocab+1)*hid = %llu does not fit the 31-bit matrix position", (2ull * cfg->vocab + 1) * ((cfg->hid + 3ull) & ~3ull));
  FV_REQUIRE(cfg->world <= MAX_RANKS, FV_ERR_INVALID, "world must be at most %d", MAX_RANKS);
  FV_REQUIRE(cfg->world >= 1 && cfg->rank >= 0 && cfg->rank < cfg->world, FV_ERR_INVALID,
             "need world >= 1 and 0 <= rank < world (rank %d, world %d)", cfg->rank, cfg->world);
  FV_REQUIRE((uint64_t)cfg->world * cfg->batch * cfg->window * (cfg->delta != 0.0f ? 2 : 1) < 0x7ffffeull, FV_ERR_INVALID,
             "world*batch*window = %llu does not fit the 23-bit scatter slot id",
             (unsigned long long)cfg->world * cfg->batch * cfg->window);
  FV_REQUIRE(cfg->delta == 0.0f || cfg->m == 2 || cfg->m == 0, FV_ERR_INVALID,
             "with delta != 0 only m = 2 (the second winner, the reference's fixed value) is implemented, got m = %u", cfg->m);
  FV_REQUIRE(cfg->delta == 0.0f || cfg->hid >= 2, FV_ERR_INVALID, "delta != 0 needs at least two hidden units");
  FV_REQUIRE(cfg->prec > 0.0f, FV_ERR_INVALID, "prec must be > 0");
  int ndev = 0;
  FV_CUDA(cudaGetDeviceCount(&ndev));
  FV_REQUIRE(cfg->device >= 0 && cfg->device < ndev, FV_ERR_INVALID, "device %d not present (%d devices)",
             cfg->device, ndev);
  int prev = 0;
  cudaGetDevice(&prev);
  fv_trainer* tr = new fv_trainer();
  const int rc = create_impl(cfg, tr);
  if (rc != FV_OK) {
    free_all(tr);
    cudaSetDevice(prev);
    return rc;
  }
  cudaSetDevice(prev);
  *out = tr;
  return FV_OK;
}

int fv_trainer_destroy(fv_trainer* tr) {
  if (!tr) return FV_OK;
  int prev = 0;
  cudaGetDevice(&prev);
  cudaSetDevice(tr->device);
  cudaDeviceSynchronize();
  free_all(tr);
  cudaSetDevice(prev);
  return FV_OK;
}

// Tokens and chunk boundaries go up once; window table and 1/count are made on the GPU.
static int pick_hot_rows(fv_trainer* tr);
static int prepare_corpus_on_device(fv_trainer* tr, const int32_t* enc, uint64_t ntok, const uint64_t* offsets,
                                    uint64_t noffsets) {
  Dev& d = tr->d;
  const unsigned long long nchunks = noffsets - 1;
  const unsigned maxlen = tr->cfg.maxlen ? tr->cfg.maxlen : 214u;
  tr->have_corpus = false;
  if (tr->d_tokens) FV_CUDA(cudaFree(tr->d_tokens));
  if (tr->d_wstart) FV_CUDA(cudaFree(tr->d_wstart));
  if (tr->d_perm) FV_CUDA(cudaFree(tr->d_perm));
  tr->d_tokens = nullptr;
  tr->d_wstart = nullptr;
  tr->d_perm = nullptr;
  unsigned long long *d_off = nullptr, *d_wbase = nullptr, *d_btot = nullptr, *d_counts = nullptr;
  uint32_t *d_nwin = nullptr, *d_err = nullptr;
  const unsigned long long nblocks = (nchunks + SCAN_BLOCK - 1) / SCAN_BLOCK;
  int rc = FV_OK;
  auto cleanup = [&]() {
    cudaFree(d_off); cudaFree(d_wbase); cudaFree(d_btot); cudaFree(d_counts); cudaFree(d_nwin); cudaFree(d_err);
  };
#define FV_PREP(expr)                                  \
  do {                                                 \
    rc = (expr);                                       \
    if (rc != FV_OK) { cleanup(); return rc; }         \
  } while (0)
#define FV_PREP_CUDA(call)                                                                                    \
  do {                                                                                                        \
    cudaError_t e_ = (call);                                                                                  \
    if (e_ != cudaSuccess) {                                                                                  \
      cleanup();                                                                                              \
      return fv::fail(FV_ERR_CUDA, "%s:%d: %s failed: %s", __FILE__, __LINE__, #call, cudaGetErrorString(e_)); \
    }                                                                                                         \
  } while (0)
  FV_PREP(dev_alloc(&tr->d_tokens, ntok));
  FV_PREP(dev_alloc(&d_off, noffsets));
  FV_PREP(dev_alloc(&d_nwin, nchunks));
  FV_PREP(dev_alloc(&d_wbase, nchunks + 1));
  FV_PREP(dev_alloc(&d_btot, 2 * nblocks));
  FV_PREP(dev_alloc(&d_counts, (size_t)d.V));
  FV_PREP(dev_alloc(&d_err, 1));
  FV_PREP_CUDA(cudaMemcpyAsync(tr->d_tokens, enc, ntok * sizeof(int32_t), cudaMemcpyHostToDevice, tr->stream));
  FV_PREP_CUDA(cudaMemcpyAsync(d_off, offsets, noffsets * sizeof(uint64_t), cudaMemcpyHostToDevice, tr->stream));
  FV_PREP_CUDA(cudaMemsetAsync(d_counts, 0, (size_t)d.V * sizeof(unsigned long long), tr->stream));
  FV_PREP_CUDA(cudaMemsetAsync(d_err, 0, sizeof(uint32_t), tr->stream));
  const int wide = tr->num_sms * 8;
  k_chunk_windows<<<wide, 256, 0, tr->stream>>>(d_off, nchunks, (unsigned)d.W, maxlen, d_nwin, d_err);
  k_block_scan<<<(unsigned)nblocks, SCAN_BLOCK, 0, tr->stream>>>(d_nwin, nchunks, nullptr, nullptr, d_btot);
  std::vector<unsigned long long> btot(nblocks), bbase(nblocks);
  FV_PREP_CUDA(cudaMemcpyAsync(btot.data(), d_btot, nblocks * sizeof(unsigned long long), cudaMemcpyDeviceToHost, tr->stream));
  FV_PREP_CUDA(cudaStreamSynchronize(tr->stream));
  unsigned long long ns = 0;
  for (unsigned long long b = 0; b < nblocks; ++b) {
    bbase[b] = ns;
    ns += btot[b];
  }
  FV_PREP_CUDA(cudaMemcpyAsync(d_btot + nblocks, bbase.data(), nblocks * sizeof(unsigned long long), cudaMemcpyHostToDevice, tr->stream));
  k_block_scan<<<(unsigned)nblocks, SCAN_BLOCK, 0, tr->stream>>>(d_nwin, nchunks, d_btot + nblocks, d_wbase, nullptr);
  FV_PREP(dev_alloc(&tr->d_wstart, ns));
  FV_PREP(dev_alloc(&tr->d_perm, ns));
  if (ns) {
    k_fill_starts<<<wide, 256, 0, tr->stream>>>(d_off, d_wbase, nchunks, ns, tr->d_wstart);
    k_iota<<<tr->num_sms * 4, 256, 0, tr->stream>>>(tr->d_perm, ns);
  }
  const size_t hist_smem = (size_t)d.V * sizeof(uint32_t);
  const int use_smem = hist_smem <= 200 * 1024;
  if (use_smem) FV_PREP_CUDA(cudaFuncSetAttribute(k_count_tokens, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)hist_smem));
  k_count_tokens<<<tr->num_sms, 512, use_smem ? hist_smem : 0, tr->stream>>>(tr->d_tokens, ntok, d.V, use_smem, d_counts, d_err);
  k_inverse_counts<<<64, 256, 0, tr->stream>>>(d_counts, d.V, (d.flags & FV_FLAG_COUNT_FP32) != 0, tr->d_f);
  FV_PREP_CUDA(cudaGetLastError());
  uint32_t err = 0;
  FV_PREP_CUDA(cudaMemcpyAsync(&err, d_err, sizeof(err), cudaMemcpyDeviceToHost, tr->stream));
  FV_PREP_CUDA(cudaStreamSynchronize(tr->stream));
  cleanup();
#undef FV_PREP
#undef FV_PREP_CUDA
  if (err & FV_DEVERR_TOKEN_RANGE) return fv::fail(FV_ERR_DATA, "a token id is >= vocab (%d)", d.V);
  if (err & FV_DEVERR_WINDOW_RANGE) return fv::fail(FV_ERR_DATA, "offsets decrease somewhere: chunk boundaries must not go backwards");
  d.tokens = tr->d_tokens;
  d.wstart = tr->d_wstart;
  d.perm = tr->d_perm;
  d.Ns = ns;
  d.ntok = ntok;
  tr->have_corpus = true;
  return pick_hot_rows(tr);
}

// Chooses the hot rows from the inverse frequencies now on the device.
static int pick_hot_rows(fv_trainer* tr) {
  const Dev& d = tr->d;
  int* d_n = nullptr;
  FV_CUDA(cudaMalloc((void**)&d_n, sizeof(int)));
  cudaMemsetAsync(tr->d_hotidx, 0xff, (size_t)d.N + 1, tr->stream);
  cudaMemsetAsync(tr->d_hot_rows, 0, HOT_ROWS * sizeof(int32_t), tr->stream);
  k_pick_hot<<<1, 1024, 0, tr->stream>>>(tr->d_f, d.V, tr->d_hotidx, tr->d_hot_rows, d_n);
  int n = 0;
  cudaError_t e = cudaGetLastError();
  if (e == cudaSuccess) e = cudaMemcpyAsync(&n, d_n, sizeof(int), cudaMemcpyDeviceToHost, tr->stream);
  if (e == cudaSuccess) e = cudaStreamSynchronize(tr->stream);
  cudaFree(d_n);
  FV_CUDA(e);
  // hot-row numbers are h (context row) and HOT_TOKENS + h (target row): the whole range is in use as soon as one token is
  tr->hot_rows_picked = n > 0 ? HOT_ROWS : 0;
  return FV_OK;
}

static int upload_corpus(fv_trainer* tr, const int32_t* enc, uint64_t ntok, const uint64_t* starts, uint64_t ns) {
  Dev& d = tr->d;
  std::vector<float> f(d.V);
  FV_TRY(fv_inverse_frequency(enc, ntok, d.V, (d.flags & FV_FLAG_COUNT_FP32) != 0, f.data()));
  tr->have_corpus = false;
  if (tr->d_tokens) FV_CUDA(cudaFree(tr->d_tokens));
  if (tr->d_wstart) FV_CUDA(cudaFree(tr->d_wstart));
  if (tr->d_perm) FV_CUDA(cudaFree(tr->d_perm));
  tr->d_tokens = nullptr;
  tr->d_wstart = nullptr;
  tr->d_perm = nullptr;
  FV_TRY(dev_alloc(&tr->d_tokens, ntok));
  FV_TRY(dev_alloc(&tr->d_wstart, ns));
  FV_TRY(dev_alloc(&tr->d_perm, ns));
  FV_CUDA(cudaMemcpyAsync(tr->d_tokens, enc, ntok * sizeof(int32_t), cudaMemcpyHostToDevice, tr->stream));
  FV_CUDA(cudaMemcpyAsync(tr->d_wstart, starts, ns * sizeof(uint64_t), cudaMemcpyHostToDevice, tr->stream));
  FV_CUDA(cudaMemcpyAsync(tr->d_f, f.data(), (size_t)d.V * sizeof(float), cudaMemcpyHostToDevice, tr->stream));
  k_iota<<<tr->num_sms * 4, 256, 0, tr->stream>>>(tr->d_perm, ns);
  FV_CUDA(cudaGetLastError());
  FV_CUDA(cudaStreamSynchronize(tr->stream));
  d.tokens = tr->d_tokens;
  d.wstart = tr->d_wstart;
  d.perm = tr->d_perm;
  d.Ns = ns;
  d.ntok = ntok;
  tr->have_corpus = true;
  return pick_hot_rows(tr);
}

int fv_trainer_set_corpus(fv_trainer* tr, const int32_t* enc, uint64_t ntok, const uint64_t* offsets,
                          uint64_t noffsets) {
  FV_REQUIRE(tr && enc && offsets, FV_ERR_INVALID, "fv_trainer_set_corpus: NULL argument");
  FV_REQUIRE(noffsets >= 2, FV_ERR_DATA, "offsets needs at least two entries");
  FV_REQUIRE(offsets[0] == 0, FV_ERR_DATA, "offsets[0] must be 0, got %llu", (unsigned long long)offsets[0]);
  FV_REQUIRE(offsets[noffsets - 1] <= ntok, FV_ERR_DATA, "last offset %llu exceeds the number of tokens %llu",
             (unsigned long long)offsets[noffsets - 1], (unsigned long long)ntok);
  fv::DeviceGuard guard(tr->device);
  FV_REQUIRE(guard.ok, FV_ERR_CUDA, "cannot select device %d", tr->device);
  return prepare_corpus_on_device(tr, enc, ntok, offsets, noffsets);
}

int fv_trainer_set_corpus_windows(fv_trainer* tr, const int32_t* enc, uint64_t ntok, const uint64_t* starts,
                                  uint64_t nwindows) {
  FV_REQUIRE(tr && enc && (starts || nwindows == 0), FV_ERR_INVALID, "fv_trainer_set_corpus_windows: NULL argument");
  for (uint64_t i = 0; i < nwindows; ++i)
    FV_REQUIRE(starts[i] + (uint64_t)tr->d.W <= ntok, FV_ERR_DATA, "window %llu starts at %llu and runs past the %llu tokens",
               (unsigned long long)i, (unsigned long long)starts[i], (unsigned long long)ntok);
  fv::DeviceGuard guard(tr->device);
  FV_REQUIRE(guard.ok, FV_ERR_CUDA, "cannot select device %d", tr->device);
  return upload_corpus(tr, enc, ntok, starts, nwindows);
}

int fv_trainer_get_window_starts(fv_trainer* tr, uint64_t* starts) {
  FV_REQUIRE(tr && starts, FV_ERR_INVALID, "fv_trainer_get_window_starts: NULL argument");
  FV_REQUIRE(tr->have_corpus, FV_ERR_STATE, "trainer has no corpus");
  fv::DeviceGuard guard(tr->device);
  FV_CUDA(cudaMemcpy(starts, tr->d_wstart, tr->d.Ns * sizeof(uint64_t), cudaMemcpyDeviceToHost));
  return FV_OK;
}

int fv_trainer_num_windows(fv_trainer* tr, uint64_t* count) {
  FV_REQUIRE(tr && count, FV_ERR_INVALID, "fv_trainer_num_windows: NULL argument");
  FV_REQUIRE(tr->have_corpus, FV_ERR_STATE, "trainer has no corpus");
  *count = tr->d.Ns;
  return FV_OK;
}

int fv_trainer_get_inverse_frequency(fv_trainer* tr, float* inv_freq) {
  FV_REQUIRE(tr && inv_freq, FV_ERR_INVALID, "fv_trainer_get_inverse_frequency: NULL argument");
  fv::DeviceGuard guard(tr->device);
  FV_CUDA(cudaMemcpy(inv_freq, tr->d_f, (size_t)tr->d.V * sizeof(float), cudaMemcpyDeviceToHost));
  return FV_OK;
}

int fv_trainer_set_inverse_frequency(fv_trainer* tr, const float* inv_freq) {
  FV_REQUIRE(tr && inv_freq, FV_ERR_INVALID, "fv_trainer_set_inverse_frequency: NULL argument");
  fv::DeviceGuard guard(tr->device);
  FV_CUDA(cudaMemcpy(tr->d_f, inv_freq, (size_t)tr->d.V * sizeof(float), cudaMemcpyHostToDevice));
  float fmax = 0.f;
  for (int v = 0; v < tr->d.V; ++v) {
    FV_REQUIRE(std::isfinite(inv_freq[v]), FV_ERR_DATA, "inverse frequency %d is not finite", v);
    fmax = std::max(fmax, std::fabs(inv_freq[v]));
  }
  tr->d.fmax = fmax;  // bounds the terms of xx (k_forward's fixed-point unit)
  return FV_OK;
}

int fv_trainer_set_weights(fv_trainer* tr, const float* w_kn) {
  FV_REQUIRE(tr && w_kn, FV_ERR_INVALID, "fv_trainer_set_weights: NULL argument");
  fv::DeviceGuard guard(tr->device);
  FV_REQUIRE(guard.ok, FV_ERR_CUDA, "cannot select device %d", tr->device);
  const Dev& d = tr->d;
  float* tmp = nullptr;
  FV_TRY(dev_alloc(&tmp, (size_t)d.K * d.N));
  cudaError_t e = cudaMemcpyAsync(tmp, w_kn, (size_t)d.K * d.N * sizeof(float), cudaMemcpyHostToDevice, tr->stream);
  if (e == cudaSuccess) {
    dim3 grid((d.N + 31) / 32, (d.Kp + 31) / 32), block(32, 8);
    k_to_device_layout<<<grid, block, 0, tr->stream>>>(tmp, tr->d_wt, d.K, d.Kp, d.N);
    k_absmax<<<tr->num_sms * 4, 256, 0, tr->stream>>>(d);
    k_reset_alpha<<<4, 256, 0, tr->stream>>>(d);
    e = cudaGetLastError();
  }
  if (e == cudaSuccess) e = cudaStreamSynchronize(tr->stream);
  cudaFree(tmp);
  FV_CUDA(e);
  tr->steps_since_fold = 0;
  tr->cand_dirty = true;
  tr->have_weights = true;
  return FV_OK;
}

int fv_trainer_get_weights(fv_trainer* tr, float* w_kn) {
  FV_REQUIRE(tr && w_kn, FV_ERR_INVALID, "fv_trainer_get_weights: NULL argument");
  FV_REQUIRE(tr->have_weights, FV_ERR_STATE, "trainer has no weights");
  fv::DeviceGuard guard(tr->device);
  FV_REQUIRE(guard.ok, FV_ERR_CUDA, "cannot select device %d", tr->device);
  const Dev& d = tr->d;
  tr->d.tick0 = tr->ticks;  // the scales of the step that would come next
  FV_TRY(fold_weights(tr, 0));
  float* tmp = nullptr;
  FV_TRY(dev_alloc(&tmp, (size_t)d.K * d.N));
  dim3 grid((d.N + 31) / 32, (d.Kp + 31) / 32), block(32, 8);
  k_to_host_layout<<<grid, block, 0, tr->stream>>>(tr->d_wt, tmp, d.K, d.Kp, d.N);
  cudaError_t e = cudaGetLastError();
  if (e == cudaSuccess)
    e = cudaMemcpyAsync(w_kn, tmp, (size_t)d.K * d.N * sizeof(float), cudaMemcpyDeviceToHost, tr->stream);
  if (e == cudaSuccess) e = cudaStreamSynchronize(tr->stream);
  cudaFree(tmp);
  FV_CUDA(e);
  return FV_OK;
}

int fv_trainer_set_permutation(fv_trainer* tr, const uint64_t* perm, uint64_t n) {
  FV_REQUIRE(tr && perm, FV_ERR_INVALID, "fv_trainer_set_permutation: NULL argument");
  FV_REQUIRE(tr->have_corpus, FV_ERR_STATE, "trainer has no corpus");
  FV_REQUIRE(n == tr->d.Ns, FV_ERR_INVALID, "permutation has %llu entries, the corpus has %llu windows",
             (unsigned long long)n, (unsigned long long)tr->d.Ns);
  fv::DeviceGuard guard(tr->device);
  FV_CUDA(cudaMemcpy(tr->d_perm, perm, n * sizeof(uint64_t), cudaMemcpyHostToDevice));
  return FV_OK;
}

int fv_trainer_shuffle(fv_trainer* tr, uint64_t seed) {
  FV_REQUIRE(tr, FV_ERR_INVALID, "fv_trainer_shuffle: NULL trainer");
  FV_REQUIRE(tr->have_corpus, FV_ERR_STATE, "trainer has no corpus");
  fv::DeviceGuard guard(tr->device);
  const unsigned long long n = tr->d.Ns;
  if (n == 0) return FV_OK;
  int bits = 1;
  while ((1ull << bits) < n) ++bits;
  int half = (bits + 1) / 2;
  if (half < 1) half = 1;
  // scramble the seed once so that nearby seeds give unrelated keys
  unsigned long long k = seed + 0x9e3779b97f4a7c15ull;
  k = (k ^ (k >> 30)) * 0xbf58476d1ce4e5b9ull;
  k = (k ^ (k >> 27)) * 0x94d049bb133111ebull;
  k ^= k >> 31;
  k_feistel_perm<<<tr->num_sms * 4, 256, 0, tr->stream>>>(tr->d_perm, n, half, k);
  FV_CUDA(cudaGetLastError());
  FV_CUDA(cudaStreamSynchronize(tr->stream));
  return FV_OK;
}

int fv_trainer_get_permutation(fv_trainer* tr, uint64_t* perm) {
  FV_REQUIRE(tr && perm, FV_ERR_INVALID, "fv_trainer_get_permutation: NULL argument");
  FV_REQUIRE(tr->have_corpus, FV_ERR_STATE, "trainer has no corpus");
  fv::DeviceGuard guard(tr->device);
  FV_CUDA(cudaMemcpy(perm, tr->d_perm, tr->d.Ns * sizeof(uint64_t), cudaMemcpyDeviceToHost));
  return FV_OK;
}

int fv_trainer_run_steps(fv_trainer* tr, uint64_t first_step, uint64_t nsteps, float eps, float* nc_out,
                         float* scale_out, fv_run_stats* stats) {
  FV_REQUIRE(tr, FV_ERR_INVALID, "fv_trainer_run_steps: NULL trainer");
  return run_steps_impl(tr, first_step, nsteps, eps, nullptr, false, nc_out, scale_out, stats);
}

int fv_trainer_run_steps_timed(fv_trainer* tr, uint64_t first_step, uint64_t nsteps, uint64_t warmup, float eps,
                               fv_run_stats* stats) {
  FV_REQUIRE(tr, FV_ERR_INVALID, "fv_trainer_run_steps_timed: NULL trainer");
  FV_REQUIRE(warmup < nsteps, FV_ERR_INVALID, "warmup (%llu) must be smaller than nsteps (%llu)", (unsigned long long)warmup,
             (unsigned long long)nsteps);
  return run_steps_impl(tr, first_step, nsteps, eps, nullptr, false, nullptr, nullptr, stats, warmup);
}

int fv_trainer_run_steps_host(fv_trainer* tr, const int32_t* idx_host, uint64_t nsteps, float eps, float* nc_out,
                              float* scale_out, fv_run_stats* stats) {
  FV_REQUIRE(tr && idx_host, FV_ERR_INVALID, "fv_trainer_run_steps_host: NULL argument");
  return run_steps_impl(tr, 0, nsteps, eps, idx_host, false, nc_out, scale_out, stats);
}

int fv_trainer_run_steps_host_local(fv_trainer* tr, const int32_t* idx_host, uint64_t nsteps, float eps, float* nc_out,
                                    float* scale_out, fv_run_stats* stats) {
  FV_REQUIRE(tr && idx_host, FV_ERR_INVALID, "fv_trainer_run_steps_host_local: NULL argument");
  return run_steps_impl(tr, 0, nsteps, eps, idx_host, true, nc_out, scale_out, stats);
}

// Learning rate of an epoch (returned) and its anti-Hebbian strength (stored in the trainer), cuda_funcs.cu:1229-1230.
static float epoch_schedule(fv_trainer* tr, uint64_t epoch, uint64_t nep) {
  // eps = lr0 * (1 - epoch/Nep): float quotient, double product, float store
  const float q = (float)epoch / (float)nep;
  const float eps = (float)((double)tr->cfg.lr0 * (1.0 - (double)q));
  // delta * 0.5 * (1 + tanh((epoch - Nep/8) / 10))
  tr->delta_now = (float)((double)tr->cfg.delta * 0.5 * (1.0 + tanh(((double)(float)epoch - 0.125 * (double)nep) / 10.0)));
  return eps;
}

// Winners [world*batch] and xx [world][K] of the last step, from this rank's copy of all ranks' packets.
static int read_packets(fv_trainer* tr, int32_t* winners, float* xx) {
  fv::DeviceGuard guard(tr->device);
  const Dev& d = tr->d;
  // the step just run had parity (ticks - 1) & 1
  const int parity = (int)((tr->ticks - 1) & 1);
  std::vector<unsigned long long> pkt((size_t)d.G * d.P);  // words: payload low, sequence number high
  FV_CUDA(cudaMemcpy(pkt.data(), tr->d_mail + MAIL_HDR + (size_t)parity * d.G * d.P * 2, pkt.size() * sizeof(unsigned long long),
                     cudaMemcpyDeviceToHost));
  for (int r = 0; r < d.G; ++r) {
    if (winners)
      for (int j = 0; j < d.B; ++j) winners[(size_t)r * d.B + j] = (int32_t)(uint32_t)pkt[(size_t)r * d.P + j];
    if (xx)
      for (int mu = 0; mu < d.K; ++mu) {
        const uint32_t bits = (uint32_t)pkt[(size_t)r * d.P + d.XO + mu];
        memcpy(xx + (size_t)r * d.K + mu, &bits, sizeof(float));
      }
  }
  return FV_OK;
}

int fv_trainer_run_epoch(fv_trainer* tr, uint64_t epoch, uint64_t nep, fv_run_stats* stats) {
  FV_REQUIRE(tr, FV_ERR_INVALID, "fv_trainer_run_epoch: NULL trainer");
  FV_REQUIRE(nep >= 1, FV_ERR_INVALID, "nep must be >= 1");
  FV_REQUIRE(tr->have_corpus, FV_ERR_STATE, "trainer has no corpus");
  const float eps = epoch_schedule(tr, epoch, nep);
  const unsigned long long per_step = (unsigned long long)tr->d.G * tr->d.B;
  const unsigned long long nsteps = (tr->d.Ns + per_step - 1) / per_step;
  return run_steps_impl(tr, 0, nsteps, eps, nullptr, false, nullptr, nullptr, stats);
}

int fv_trainer_step_debug(fv_trainer* tr, uint64_t step, float eps, int32_t* winners, float* xx, float* nc,
                          float* scale) {
  FV_REQUIRE(tr, FV_ERR_INVALID, "fv_trainer_step_debug: NULL trainer");
  float nc1 = 0.f, s1 = 0.f;
  FV_TRY(run_steps_impl(tr, step, 1, eps, nullptr, false, &nc1, &s1, nullptr));
  FV_TRY(read_packets(tr, winners, xx));
  if (nc) *nc = nc1;
  if (scale) *scale = s1;
  return FV_OK;
}

int fv_trainer_time_forward(fv_trainer* tr, uint64_t step, uint32_t reps, double* seconds_per_launch) {
  FV_REQUIRE(tr && seconds_per_launch && reps >= 1, FV_ERR_INVALID, "fv_trainer_time_forward: bad argument");
  FV_REQUIRE(tr->have_weights && tr->have_corpus, FV_ERR_STATE, "trainer needs a corpus and weights");
  fv::DeviceGuard guard(tr->device);
  FV_REQUIRE(guard.ok, FV_ERR_CUDA, "cannot select device %d", tr->device);
  const Dev& d = tr->d;
  const size_t step_ids = (size_t)d.G * d.B * d.W;
  if (!tr->d_idx_stage[0]) FV_TRY(dev_alloc(&tr->d_idx_stage[0], step_ids * STAGE_STEPS));
  tr->d.tick0 = tr->ticks;
  k_set_ctl<<<1, 1, 0, tr->stream>>>(tr->d_ctl, step, 0.f, tr->delta_now);
  k_build_idx_block<<<tr->num_sms * 4, 256, 0, tr->stream>>>(d, step, 1, tr->d_idx_stage[0]);
  // the kernel only writes winners and adds to the xx accumulators, so it can be repeated on the same
  // step; alternating the parity lets each launch clear the ticket counter of the next.  The launches
  // keep their winners to this rank: a peer must not find words of a step that never ran.
  uint32_t* const* const peers = tr->d.peers;
  tr->d.peers = nullptr;
  tr->d.nhot = 0;  // nobody would collect the counts; the next step loop sets it again
  for (uint32_t r = 0; r < 3; ++r) FV_DISPATCH_NT(tr->NT, launch_forward, tr, (int)(r & 1), tr->d_idx_stage[0]);
  FV_CUDA(cudaEventRecord(tr->ev_begin, tr->stream));
  for (uint32_t r = 0; r < reps; ++r) FV_DISPATCH_NT(tr->NT, launch_forward, tr, (int)((r + 1) & 1), tr->d_idx_stage[0]);
  FV_CUDA(cudaEventRecord(tr->ev_end, tr->stream));
  tr->d.peers = peers;
  // no xx_finish ran: clear what the launches added to the accumulators
  FV_CUDA(cudaMemsetAsync(tr->d_xx_acc, 0, 2 * (size_t)XX_SLOTS * d.Kp * sizeof(unsigned long long), tr->stream));
  FV_CUDA(cudaMemsetAsync(tr->d_xx_wins, 0, (size_t)d.Kp * sizeof(uint32_t), tr->stream));
  FV_CUDA(cudaGetLastError());
  FV_CUDA(cudaStreamSynchronize(tr->stream));
  float ms = 0.f;
  FV_CUDA(cudaEventElapsedTime(&ms, tr->ev_begin, tr->ev_end));
  *seconds_per_launch = ms * 1e-3 / reps;
  return FV_OK;
}

int fv_comm_unique_id(uint8_t id[128]) {
  FV_REQUIRE(id, FV_ERR_INVALID, "fv_comm_unique_id: NULL id");
  FV_TRY(load_nccl());
  Id128 uid;
  memset(&uid, 0, sizeof(uid));
  const int rc = g_nccl.GetUniqueId(&uid);
  if (rc != 0) return fv::fail(FV_ERR_COMM, "ncclGetUniqueId failed: %s", g_nccl.GetErrorString(rc));
  memcpy(id, uid.bytes, 128);
  return FV_OK;
}

int fv_trainer_init_comm(fv_trainer* tr, const uint8_t id[128]) {
  FV_REQUIRE(tr && id, FV_ERR_INVALID, "fv_trainer_init_comm: NULL argument");
  if (tr->d.G == 1) return FV_OK;
  FV_REQUIRE(tr->comm == nullptr, FV_ERR_STATE, "communicator already initialised");
  FV_TRY(load_nccl());
  fv::DeviceGuard guard(tr->device);
  FV_REQUIRE(guard.ok, FV_ERR_CUDA, "cannot select device %d", tr->device);
  Id128 uid;
  memcpy(uid.bytes, id, 128);
  void* comm = nullptr;
  int rc = g_nccl.CommInitRank(&comm, tr->d.G, uid, tr->d.rank);
  if (rc != 0) return fv::fail(FV_ERR_COMM, "ncclCommInitRank failed: %s", g_nccl.GetErrorString(rc));
  tr->comm = comm;
  tr->comm_mode = 1;

  // Peer-memory mailboxes: every rank exports its mailbox, the handles travel through the
  // communicator just created, every rank maps the others'.  If any rank cannot (no peer
  // access between the GPUs, handle not importable), all ranks stay with the all-gather.
  const char* force = getenv("FV_COMM");
  const int G = tr->d.G;
  constexpr int HB = (int)sizeof(cudaIpcMemHandle_t);  // 64 bytes
  static_assert(sizeof(cudaIpcMemHandle_t) % 4 == 0, "handle size");
  int ok = (force && strcmp(force, "nccl") == 0) ? 0 : 1;
  cudaIpcMemHandle_t mine;
  memset(&mine, 0, sizeof(mine));
  if (ok && cudaIpcGetMemHandle(&mine, tr->d_mail) != cudaSuccess) {
    cudaGetLastError();
    ok = 0;
  }
  uint32_t* d_ex = nullptr;  // [G][HB/4 + 1]: handle words, then an "ok" word
  const int words = HB / 4 + 1;
  FV_TRY(dev_alloc(&d_ex, (size_t)G * words));
  std::vector<uint32_t> ex((size_t)G * words, 0u);
  memcpy(ex.data() + (size_t)tr->d.rank * words, &mine, HB);
  ex[(size_t)tr->d.rank * words + HB / 4] = (uint32_t)ok;
  cudaError_t e = cudaMemcpyAsync(d_ex, ex.data(), ex.size() * 4, cudaMemcpyHostToDevice, tr->stream);
  if (e == cudaSuccess) {
    rc = g_nccl.AllGather(d_ex + (size_t)tr->d.rank * words, d_ex, (size_t)words, NCCL_UINT32, tr->comm, tr->stream);
    if (rc != 0) {
      cudaFree(d_ex);
      return fv::fail(FV_ERR_COMM, "ncclAllGather (handles) failed: %s", g_nccl.GetErrorString(rc));
    }
    e = cudaMemcpyAsync(ex.data(), d_ex, ex.size() * 4, cudaMemcpyDeviceToHost, tr->stream);
  }
  if (e == cudaSuccess) e = cudaStreamSynchronize(tr->stream);
  if (e != cudaSuccess) {
    cudaFree(d_ex);
    FV_CUDA(e);
  }
  int all_ok = 1;
  for (int r = 0; r < G; ++r) all_ok &= (int)ex[(size_t)r * words + HB / 4];
  int mapped = all_ok;
  if (all_ok) {
    for (int r = 0; r < G && mapped; ++r) {
      if (r == tr->d.rank) {
        tr->peer_mail[r] = tr->d_mail;
        continue;
      }
      cudaIpcMemHandle_t hnd;
      memcpy(&hnd, ex.data() + (size_t)r * words, HB);
      void* p = nullptr;
      if (cudaIpcOpenMemHandle(&p, hnd, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) {
        cudaGetLastError();
        mapped = 0;
      } else {
        tr->peer_mail[r] = static_cast<uint32_t*>(p);
      }
    }
  }
  // second round: did everybody manage to map everybody?
  ex.assign((size_t)G * words, 0u);
  ex[(size_t)tr->d.rank * words] = (uint32_t)mapped;
  e = cudaMemcpyAsync(d_ex, ex.data(), ex.size() * 4, cudaMemcpyHostToDevice, tr->stream);
  if (e == cudaSuccess) {
    rc = g_nccl.AllGather(d_ex + (size_t)tr->d.rank * words, d_ex, (size_t)words, NCCL_UINT32, tr->comm, tr->stream);
    if (rc != 0) {
      cudaFree(d_ex);
      return fv::fail(FV_ERR_COMM, "ncclAllGather (mapping) failed: %s", g_nccl.GetErrorString(rc));
    }
    e = cudaMemcpyAsync(ex.data(), d_ex, ex.size() * 4, cudaMemcpyDeviceToHost, tr->stream);
  }
  if (e == cudaSuccess) e = cudaStreamSynchronize(tr->stream);
  cudaFree(d_ex);
  FV_CUDA(e);
  int all_mapped = 1;
  for (int r = 0; r < G; ++r) all_mapped &= (int)ex[(size_t)r * words];
  if (all_mapped) {
    FV_TRY(dev_alloc(&tr->d_peer_table, (size_t)MAX_RANKS));
    FV_CUDA(cudaMemcpy(tr->d_peer_table, tr->peer_mail, sizeof(uint32_t*) * MAX_RANKS, cudaMemcpyHostToDevice));
    tr->d.peers = tr->d_peer_table;
    tr->comm_mode = 2;
    tr->d.shard = default_shard(tr);
    tr->cand_dirty = true;
  } else {
    for (int r = 0; r < G; ++r) {
      if (tr->peer_mail[r] && r != tr->d.rank) cudaIpcCloseMemHandle(tr->peer_mail[r]);
      tr->peer_mail[r] = nullptr;
    }
  }
  return FV_OK;
}

int fv_trainer_set_option(fv_trainer* tr, const char* key, double value) {
  FV_REQUIRE(tr && key, FV_ERR_INVALID, "fv_trainer_set_option: NULL argument");
  if (strcmp(key, "spin_limit") == 0) {
    FV_REQUIRE(value >= 1.0 && value <= 4.0e9, FV_ERR_INVALID, "spin_limit must be in [1, 4e9], got %g", value);
    tr->d.spin_limit = (unsigned)value;
    return FV_OK;
  }
  if (strcmp(key, "tag_variant") == 0) {
    FV_REQUIRE(value == 0.0 || value == 1.0 || value == 2.0 || value == 3.0, FV_ERR_INVALID, "tag_variant must be 0 (by size), 1, 2 or 3, got %g", value);
    choose_tag_variant(tr, (int)value);
    return FV_OK;
  }
  if (strcmp(key, "tag_slots") == 0) {
    FV_REQUIRE(value == 0.0 || value == 1.0 || value == 2.0 || value == 4.0 || value == 8.0, FV_ERR_INVALID,
               "tag_slots must be 0 (by size), 1, 2, 4 or 8, got %g", value);
    choose_tag_variant(tr, 0);
    if (value != 0.0) {
      const size_t E = (size_t)tr->d.G * tr->d.B * tr->d.W * (1 + tr->d.has_delta);
      tr->tag_batch_u = (int)value;
      tr->tag_batch_grid = grid_for(E, XX_THREADS * tr->tag_batch_u, tr->num_sms * 3 - 1 - PUSH_CTAS - HOT_PUSH_CTAS);
    }
    return FV_OK;
  }
  if (strcmp(key, "fused_update") == 0) {
    FV_REQUIRE(value == 0.0 || value == 1.0, FV_ERR_INVALID, "fused_update must be 0 or 1, got %g", value);
    tr->fused_update = value != 0.0;
    return FV_OK;
  }
  if (strcmp(key, "hot_pairs") == 0) {
    FV_REQUIRE(value == 0.0 || value == 1.0, FV_ERR_INVALID, "hot_pairs must be 0 or 1, got %g", value);
    tr->hot_pairs = value != 0.0;
    return FV_OK;
  }
  if (strcmp(key, "colmax_lists") == 0) {
    FV_REQUIRE(value == 0.0 || value == 1.0, FV_ERR_INVALID, "colmax_lists must be 0 or 1, got %g", value);
    tr->d.use_cand = (int)value;
    tr->cand_dirty = true;
    return FV_OK;
  }
  if (strcmp(key, "shard") == 0) {
    FV_REQUIRE(value == 0.0 || value == 1.0, FV_ERR_INVALID, "shard must be 0 or 1, got %g", value);
    FV_REQUIRE(value == 0.0 || (tr->comm_mode == 2 && !tr->d.has_delta), FV_ERR_STATE,
               "the sharded update needs peer mailboxes (fv_trainer_init_comm or fv_trainers_link first) and delta == 0");
    tr->d.shard = (int)value;
    tr->cand_dirty = true;  // the candidate lists cover the rows a rank scans: all rows, or the ones it owns
    return FV_OK;
  }
  if (strcmp(key, "loopback_peers") == 0) {
    // Test aid: every peer's mailbox is this rank's own, so nothing a peer would send ever arrives and
    // the first wait for a peer's word runs into spin_limit.
    FV_REQUIRE(value == 1.0 && tr->d.G > 1 && tr->comm_mode == 0, FV_ERR_STATE, "loopback_peers: needs world > 1 and no communicator yet");
    fv::DeviceGuard guard(tr->device);
    for (int r = 0; r < tr->d.G; ++r) tr->peer_mail[r] = tr->d_mail;
    FV_TRY(dev_alloc(&tr->d_peer_table, (size_t)MAX_RANKS));
    FV_CUDA(cudaMemcpy(tr->d_peer_table, tr->peer_mail, sizeof(uint32_t*) * MAX_RANKS, cudaMemcpyHostToDevice));
    tr->d.peers = tr->d_peer_table;
    tr->linked = true;
    tr->comm_mode = 2;
    return FV_OK;
  }
  return fv::fail(FV_ERR_INVALID, "fv_trainer_set_option: unknown option %s", key);
}

// ---------------------------------------------------------------------------
// Several ranks driven by one process
// ---------------------------------------------------------------------------
int fv_trainers_link(fv_trainer* const* trs, int32_t n) {
  FV_REQUIRE(trs && n >= 1 && n <= MAX_RANKS, FV_ERR_INVALID, "fv_trainers_link: need 1..%d trainers", MAX_RANKS);
  bool same_device = true, distinct = true;
  for (int r = 0; r < n; ++r) {
    FV_REQUIRE(trs[r], FV_ERR_INVALID, "fv_trainers_link: trainer %d is NULL", r);
    const fv_config &a = trs[r]->cfg, &b = trs[0]->cfg;
    FV_REQUIRE(a.world == n && a.rank == r, FV_ERR_INVALID, "fv_trainers_link: trainer %d has rank %d of %d, expected rank %d of %d", r,
               a.rank, a.world, r, n);
    FV_REQUIRE(a.hid == b.hid && a.vocab == b.vocab && a.window == b.window && a.batch == b.batch && a.delta == b.delta &&
                   a.flags == b.flags && a.prec == b.prec,
               FV_ERR_INVALID, "fv_trainers_link: trainer %d is configured differently from trainer 0", r);
    FV_REQUIRE(trs[r]->comm_mode == 0, FV_ERR_STATE, "fv_trainers_link: trainer %d already has a communicator", r);
    FV_REQUIRE(!(a.flags & FV_FLAG_EMULATE_RANKS), FV_ERR_INVALID, "fv_trainers_link: FV_FLAG_EMULATE_RANKS computes all ranks in one trainer");
    same_device &= trs[r]->device == trs[0]->device;
    for (int q = 0; q < r; ++q) distinct &= trs[q]->device != trs[r]->device;
  }
  if (n == 1) return FV_OK;
  FV_REQUIRE(same_device || distinct, FV_ERR_INVALID, "fv_trainers_link: the trainers must sit on %d different devices, or all on one", n);
  if (distinct) {
    for (int r = 0; r < n; ++r) {
      fv::DeviceGuard guard(trs[r]->device);
      FV_REQUIRE(guard.ok, FV_ERR_CUDA, "cannot select device %d", trs[r]->device);
      for (int q = 0; q < n; ++q) {
        if (q == r) continue;
        int can = 0;
        FV_CUDA(cudaDeviceCanAccessPeer(&can, trs[r]->device, trs[q]->device));
        FV_REQUIRE(can, FV_ERR_COMM, "device %d cannot access the memory of device %d", trs[r]->device, trs[q]->device);
        const cudaError_t e = cudaDeviceEnablePeerAccess(trs[q]->device, 0);
        if (e == cudaErrorPeerAccessAlreadyEnabled) cudaGetLastError();
        else FV_CUDA(e);
      }
    }
  }
  for (int r = 0; r < n; ++r) {
    fv_trainer* tr = trs[r];
    fv::DeviceGuard guard(tr->device);
    for (int q = 0; q < n; ++q) tr->peer_mail[q] = trs[q]->d_mail;
    FV_TRY(dev_alloc(&tr->d_peer_table, (size_t)MAX_RANKS));
    FV_CUDA(cudaMemcpy(tr->d_peer_table, tr->peer_mail, sizeof(uint32_t*) * MAX_RANKS, cudaMemcpyHostToDevice));
    tr->d.peers = tr->d_peer_table;
    tr->linked = true;
    tr->comm_mode = 2;
    tr->d.shard = default_shard(tr);
    tr->cand_dirty = true;
    if (same_device) {
      tr->lockstep = true;
      if (r > 0) {
        FV_CUDA(cudaStreamSynchronize(tr->stream));
        FV_CUDA(cudaStreamDestroy(tr->stream));
        tr->stream = trs[0]->stream;
        tr->own_stream = false;
      }
    }
  }
  return FV_OK;
}

static int run_group(fv_trainer* const* trs, int n, unsigned long long first_step, unsigned long long nsteps, float eps,
                     unsigned long long timed_from, float* nc_out, float* scale_out, fv_run_stats* stats) {
  FV_REQUIRE(trs && n >= 1, FV_ERR_INVALID, "NULL trainer list");
  for (int r = 0; r < n; ++r)
    FV_REQUIRE(trs[r] && trs[r]->d.G == n && trs[r]->d.rank == r && (n == 1 || trs[r]->linked), FV_ERR_STATE,
               "the trainers must be ranks 0..%d of one linked group, in order", n - 1);
  if (nsteps == 0) return FV_OK;
  if (n == 1) return run_steps_impl(trs[0], first_step, nsteps, eps, nullptr, false, nc_out, scale_out, stats, timed_from);
  if (trs[0]->lockstep) {
    // one device, one stream: every phase of a step for rank 0, 1, ... before the next phase, so that
    // whatever a kernel waits for has been written by a kernel that is already complete
    fv::DeviceGuard guard(trs[0]->device);
    FV_REQUIRE(guard.ok, FV_ERR_CUDA, "cannot select device %d", trs[0]->device);
    std::vector<StepLoop> L(n);
    for (int r = 0; r < n; ++r) {
      L[r].first_step = first_step;
      L[r].nsteps = nsteps;
      L[r].eps = eps;
      L[r].timed_from = timed_from;
      FV_TRY(loop_begin(trs[r], L[r]));
    }
    // FV_LOCKSTEP_TIMES=1: time every phase of rank 0 with an event pair (the ranks run one after the other
    // here, so these are a rank's own kernel times with nothing to wait for); printed to stderr
    const bool timing = getenv("FV_LOCKSTEP_TIMES") != nullptr;
    std::vector<cudaEvent_t> evs;
    for (unsigned long long k = 0; k < nsteps; ++k) {
      for (int r = 0; r < n; ++r) FV_TRY(loop_stage(trs[r], L[r], k));
      for (int ph = 0; ph < STEP_PHASES; ++ph)
        for (int r = 0; r < n; ++r) {
          const bool mark = timing && r == 0 && k >= timed_from;
          if (mark) {
            evs.emplace_back();
            FV_CUDA(cudaEventCreate(&evs.back()));
            FV_CUDA(cudaEventRecord(evs.back(), trs[0]->stream));
          }
          FV_TRY(enqueue_phase(trs[r], ph, (int)k, L[r].idx, &L[r].launches));
          if (mark) {
            evs.emplace_back();
            FV_CUDA(cudaEventCreate(&evs.back()));
            FV_CUDA(cudaEventRecord(evs.back(), trs[0]->stream));
          }
        }
      for (int r = 0; r < n; ++r) FV_TRY(loop_after_step(trs[r], L[r], k));
    }
    if (timing && !evs.empty()) {
      FV_CUDA(cudaStreamSynchronize(trs[0]->stream));
      double sum[STEP_PHASES] = {0};
      for (size_t e = 0; e + 1 < evs.size(); e += 2) {
        float ms = 0.f;
        cudaEventElapsedTime(&ms, evs[e], evs[e + 1]);
        sum[(e / 2) % STEP_PHASES] += ms;
      }
      const double steps_timed = (double)(evs.size() / 2 / STEP_PHASES);
      fprintf(stderr, "[lockstep, rank 0 alone] us per step: forward %.1f exchange %.1f tag %.1f scan %.1f apply %.1f\n",
              sum[0] * 1e3 / steps_timed, sum[1] * 1e3 / steps_timed, sum[2] * 1e3 / steps_timed, sum[3] * 1e3 / steps_timed,
              sum[4] * 1e3 / steps_timed);
      for (cudaEvent_t e : evs) cudaEventDestroy(e);
    }
    int rc = FV_OK;
    for (int r = 0; r < n; ++r) {
      const int e = loop_end(trs[r], L[r], r == 0 ? nc_out : nullptr, r == 0 ? scale_out : nullptr, stats ? stats + r : nullptr);
      if (e != FV_OK && rc == FV_OK) rc = e;
    }
    return rc;
  }
  // one device per rank: a host thread each, as the reference drives its GPUs (cuda_funcs.cu:1664-1665)
  std::vector<int> rcs(n, FV_OK);
  std::vector<std::string> msgs(n);
#pragma omp parallel for num_threads(n) schedule(static, 1)
  for (int r = 0; r < n; ++r) {
    rcs[r] = run_steps_impl(trs[r], first_step, nsteps, eps, nullptr, false, r == 0 ? nc_out : nullptr, r == 0 ? scale_out : nullptr,
                            stats ? stats + r : nullptr, timed_from);
    if (rcs[r] != FV_OK) msgs[r] = fv_last_error();
  }
  for (int r = 0; r < n; ++r)
    if (rcs[r] != FV_OK) return fv::fail(rcs[r], "rank %d: %s", r, msgs[r].c_str());
  return FV_OK;
}

int fv_trainers_run_steps(fv_trainer* const* trs, int32_t n, uint64_t first_step, uint64_t nsteps, uint64_t warmup, float eps,
                          float* nc_out, float* scale_out, fv_run_stats* stats) {
  FV_REQUIRE(nsteps == 0 || warmup < nsteps, FV_ERR_INVALID, "warmup must be smaller than nsteps");
  return run_group(trs, n, first_step, nsteps, eps, warmup, nc_out, scale_out, stats);
}

int fv_trainers_run_epoch(fv_trainer* const* trs, int32_t n, uint64_t epoch, uint64_t nep, fv_run_stats* stats) {
  FV_REQUIRE(trs && n >= 1 && trs[0], FV_ERR_INVALID, "fv_trainers_run_epoch: NULL trainer list");
  FV_REQUIRE(nep >= 1, FV_ERR_INVALID, "nep must be >= 1");
  FV_REQUIRE(trs[0]->have_corpus, FV_ERR_STATE, "trainer has no corpus");
  float eps = 0.f;
  for (int r = 0; r < n; ++r) {
    FV_REQUIRE(trs[r], FV_ERR_INVALID, "fv_trainers_run_epoch: trainer %d is NULL", r);
    eps = epoch_schedule(trs[r], epoch, nep);
  }
  const unsigned long long per_step = (unsigned long long)trs[0]->d.G * trs[0]->d.B;
  const unsigned long long nsteps = (trs[0]->d.Ns + per_step - 1) / per_step;
  return run_group(trs, n, 0, nsteps, eps, 0, nullptr, nullptr, stats);
}

int fv_trainer_last_packets(fv_trainer* tr, int32_t* winners, float* xx) {
  FV_REQUIRE(tr, FV_ERR_INVALID, "fv_trainer_last_packets: NULL trainer");
  FV_REQUIRE(tr->ticks > 0, FV_ERR_STATE, "no step has run yet");
  return read_packets(tr, winners, xx);
}

int fv_trainer_get_counter(fv_trainer* tr, const char* key, uint64_t* value) {
  FV_REQUIRE(tr && key && value, FV_ERR_INVALID, "fv_trainer_get_counter: NULL argument");
  if (strcmp(key, "matrix_scans") == 0) {
    *value = tr->matrix_scans;
    return FV_OK;
  }
  if (strcmp(key, "column_rescans") == 0) {
    *value = tr->column_rescans;
    return FV_OK;
  }
  return fv::fail(FV_ERR_INVALID, "fv_trainer_get_counter: unknown counter %s", key);
}

int fv_trainer_comm_mode(fv_trainer* tr, int* mode) {
  FV_REQUIRE(tr && mode, FV_ERR_INVALID, "fv_trainer_comm_mode: NULL argument");
  *mode = tr->comm_mode;
  return FV_OK;
}

}  // extern "C"
