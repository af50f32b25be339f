/*
 * flyvec_b200 -- C ABI of the B200-native FlyVec trainer and hasher.
 *
 * Plain pointers and sizes only; every call returns an fv_status and never
 * exits the process.  After a non-zero status fv_last_error() holds a message
 * for the calling thread.  One trainer handle drives one GPU (one data-parallel
 * rank); calls on one handle must not overlap.
 *
 * Each group below names the reference interface it stands in for
 * (paths relative to the bhoov/flyvec project root).
 */
#ifndef FLYVEC_B200_H
#define FLYVEC_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define FV_ABI_VERSION 1

typedef enum fv_status {
  FV_OK = 0,
  FV_ERR_INVALID = 1, /* bad argument or configuration                       */
  FV_ERR_CUDA = 2,    /* a CUDA runtime call failed                          */
  FV_ERR_COMM = 3,    /* NCCL missing or a collective failed                 */
  FV_ERR_STATE = 4,   /* call made before its prerequisites (corpus, ...)    */
  FV_ERR_DATA = 5,    /* input data violate the format (token id >= V, ...)  */
  FV_ERR_TIMEOUT = 6  /* a bounded device-side wait ran out                  */
} fv_status;

/* ---- flags --------------------------------------------------------------- */
#define FV_FLAG_COUNT_FP32 1u      /* word counts saturate at 2^24 like the reference's float counters */
#define FV_FLAG_ACC_FP64 2u        /* forward pass accumulates every unit in double (slower, same result) */
#define FV_FLAG_FOLD_EVERY_STEP 4u /* fold the per-unit scale into the weights after every step */
#define FV_FLAG_EMULATE_RANKS 8u   /* one process computes the blocks of all `world` ranks in turn and skips the
                                      exchange: the cross-rank combine on a single GPU, for tests */

#define FV_HASH_PACKED 0u   /* output ceil(K/8) bytes per item, unit mu = bit mu%8 of byte mu/8 */
#define FV_HASH_BYTES 1u    /* output K bytes per item, each 0 or 1 (the reference's int8 layout) */
#define FV_HASH_RAW 2u      /* window hashing: unweighted activation (the form training selects on) */
#define FV_HASH_NO_UNK 4u   /* token hashing: do not zero the code of id 0 */
#define FV_HASH_EXACT 8u    /* window hashing: sum every window in double like the reference, without the
                               certified float pass (same codes, slower; for checks) */

/*
 * Hyper-parameters of one trainer.  Stands in for the reference's
 * model_descriptor and its string-keyed setters
 * (flyvec/src/model_descriptor.h:13-66, flyvec/src/model_descriptor.cu:50-112,
 * pushed from flyvec/train_flyvec.py:191-213).
 */
typedef struct fv_config {
  uint32_t struct_size; /* sizeof(fv_config), checked                          */
  int32_t device;       /* CUDA device ordinal                                 */
  int32_t rank;         /* data-parallel rank, 0 <= rank < world               */
  int32_t world;        /* number of ranks (GPUs); 1 = single GPU              */
  uint32_t hid;         /* K, number of hidden units        ("hid")            */
  uint32_t vocab;       /* V, vocabulary size; N = 2V       ("vocabulary_size")*/
  uint32_t window;      /* W, window length incl. the centre ("W")             */
  uint32_t batch;       /* windows per GPU per step         ("Num")            */
  float lr0;            /* initial learning rate  ("initial_learning_rate")    */
  float delta;          /* anti-Hebbian strength  ("delta"); run_epoch applies the epoch schedule */
  float prec;           /* lower bound of the normaliser ("prec")              */
  uint32_t m;           /* rank of the anti-Hebbian unit ("m", 2 in the reference) */
  uint32_t maxlen;      /* chunks this long or longer are dropped; 0 -> 214    */
  uint32_t flags;       /* FV_FLAG_*                                           */
} fv_config;

/* Timing and diagnostics of one fv_trainer_run_* call. */
typedef struct fv_run_stats {
  uint64_t steps;          /* global minibatch steps executed                  */
  uint64_t windows;        /* windows this rank processed                      */
  double seconds;          /* device time of the step loop (CUDA events)       */
  /* the next three come from a clock the kernels keep on the device (whole run) */
  double fwd_seconds;      /* the fused gather/arg-max kernel                  */
  double exch_seconds;     /* xx kernel + all-gather (comm mode 1 only)        */
  double upd_seconds;      /* scatter bookkeeping (with any wait for a peer's
                              words, comm mode 2), abs-max scan, update        */
  uint64_t kernel_launches;/* kernels of this library launched in the loop     */
  float last_nc;           /* normaliser of the last step                      */
  float last_scale;        /* eps / max(prec, nc) of the last step             */
  uint32_t device_error;   /* non-zero: a bounds predicate fired on the device */
  uint32_t timed_steps;    /* steps between the two timing events (`seconds`, `windows` and the three
                              phase times cover these; all steps unless the call named a warm-up)     */
} fv_run_stats;

typedef struct fv_trainer fv_trainer;
typedef struct fv_hasher fv_hasher;

/* ---- library ------------------------------------------------------------- */
int fv_version(void);
const char* fv_last_error(void);
/* cuda_helpers.cu:31-35 get_cuda_num_devices */
int fv_device_count(int* count);

/* ---- corpus preparation (host) -------------------------------------------
 * prune_input.cpp:63-84 getnum_samples and 87-122 compute_offset_phrases:
 * windows of `window` tokens that stay inside one chunk; chunks shorter than
 * the window or of `maxlen` tokens and more are dropped.  `offsets` has
 * nchunks+1 entries, offsets[0] == 0, last entry == number of tokens.
 * Pass starts == NULL to count only.
 */
int fv_enumerate_windows(const uint64_t* offsets, uint64_t nchunks, uint32_t window, uint32_t maxlen,
                         uint64_t* count, uint64_t* starts);
/* model_arrays.cu:395-424 compute_inverse_word_frequency: f[v] = 1/count(v),
 * 0 for unseen ids, negative ids skipped; saturate != 0 caps counts at 2^24. */
int fv_inverse_frequency(const int32_t* enc, uint64_t ntok, uint32_t vocab, int saturate, float* inv_freq);

/* ---- trainer -------------------------------------------------------------
 * model_create_descriptor / model_create_arrays / model_arrays_allocate_memory
 * (model_descriptor.cu:17-48, model_arrays.cu:14-40); the library owns all
 * device memory and frees it in fv_trainer_destroy.
 */
int fv_trainer_create(const fv_config* cfg, fv_trainer** out);
int fv_trainer_destroy(fv_trainer* tr);

/* Stands in for the pinned INPUT buffer, set_up_INPUT_pointer and
 * compute_inverse_word_frequency (train_flyvec.py:155-185, 223-229): copies the
 * token ids and chunk boundaries to the GPU and builds the window table and 1/count there. */
int fv_trainer_set_corpus(fv_trainer* tr, const int32_t* enc, uint64_t ntok, const uint64_t* offsets,
                          uint64_t noffsets);
/* The same with the window table already made (what compute_offset_phrases produced,
 * prune_input.cpp:87-122, and set_up_INPUT_pointer consumed, model_arrays.cu:357-393). */
int fv_trainer_set_corpus_windows(fv_trainer* tr, const int32_t* enc, uint64_t ntok, const uint64_t* starts,
                                  uint64_t nwindows);
int fv_trainer_num_windows(fv_trainer* tr, uint64_t* count);
/* The window table as built on the GPU (what compute_offset_phrases writes, prune_input.cpp:87-122). */
int fv_trainer_get_window_starts(fv_trainer* tr, uint64_t* starts /* [num_windows] */);
int fv_trainer_get_inverse_frequency(fv_trainer* tr, float* inv_freq /* [V] */);
int fv_trainer_set_inverse_frequency(fv_trainer* tr, const float* inv_freq /* [V] */);

/* get_data_pointer("synapses") + numpy.copyto (train_flyvec.py:245-250): the
 * host layout is the checkpoint layout, float32 [K][2V] C-order. */
int fv_trainer_set_weights(fv_trainer* tr, const float* w_kn);
int fv_trainer_get_weights(fv_trainer* tr, float* w_kn);

/* do_reshuffle_indices (model_arrays.cu:441-465).  The reference's quasi-random
 * transposition shuffle cannot be reproduced from outside, so the order of the
 * windows is either given explicitly or drawn from a seed (a keyed bijection
 * of [0, Ns) evaluated on the GPU). */
int fv_trainer_set_permutation(fv_trainer* tr, const uint64_t* perm, uint64_t n);
int fv_trainer_shuffle(fv_trainer* tr, uint64_t seed);
int fv_trainer_get_permutation(fv_trainer* tr, uint64_t* perm /* [Ns] */);

/* launch_epoch_INPUT_AS_INT (cuda_funcs.cu:1219-1257): eps = lr0*(1-epoch/nep),
 * then every minibatch of the current window order. */
int fv_trainer_run_epoch(fv_trainer* tr, uint64_t epoch, uint64_t nep, fv_run_stats* stats);
/* A slice of run_epoch's loop (cuda_funcs.cu:1662-1812): global steps
 * [first_step, first_step+nsteps) at a given eps.  nc_out / scale_out, when not
 * NULL, receive nsteps values each (the per-step normaliser and step size). */
int fv_trainer_run_steps(fv_trainer* tr, uint64_t first_step, uint64_t nsteps, float eps, float* nc_out,
                         float* scale_out, fv_run_stats* stats);
/* The same with the first `warmup` steps outside the timed region: the timing event is recorded on the
 * stream between step warmup-1 and step warmup, so stats->seconds, ->windows and the phase times cover
 * steps [warmup, nsteps) of a loop that is already in its steady state. */
int fv_trainer_run_steps_timed(fv_trainer* tr, uint64_t first_step, uint64_t nsteps, uint64_t warmup, float eps,
                               fv_run_stats* stats);
/* Same loop fed from host memory: idx_host holds nsteps*world*batch windows of
 * `window` pre-built input ids (token, centre token + V, or -1), uploaded inside
 * the call; per-step normalisers are copied back.  This is the streaming form
 * of the reference's zero-copy reads of pinned host tokens (cuda_funcs.cu:1679-1680). */
int fv_trainer_run_steps_host(fv_trainer* tr, const int32_t* idx_host, uint64_t nsteps, float eps, float* nc_out,
                              float* scale_out, fv_run_stats* stats);
/* The same with every rank passing only ITS OWN windows (nsteps*batch of them, in step order): the
 * ranks' ids meet on the GPUs through an all-gather over NVLink that runs a block of steps ahead on a
 * second stream, so a rank uploads 1/world of what fv_trainer_run_steps_host takes.  With one rank
 * the two calls are the same. */
int fv_trainer_run_steps_host_local(fv_trainer* tr, const int32_t* idx_host, uint64_t nsteps, float eps, float* nc_out,
                                    float* scale_out, fv_run_stats* stats);
/* One step with its intermediates copied out, for parity checks:
 * winners[world*batch] (-1 for absent windows), xx[world][K], nc, scale. */
int fv_trainer_step_debug(fv_trainer* tr, uint64_t step, float eps, int32_t* winners, float* xx, float* nc,
                          float* scale);

/* Measurement aid: average duration of the fused gather/arg-max kernel (T4-T8 for this rank's block of
 * global step `step`) over `reps` back-to-back launches, timed with CUDA events on the trainer's stream.
 * The kernel only writes winners and xx terms, so repeating it leaves the weights untouched; the launches keep
 * their winners to this rank (nothing is sent to peers). */
int fv_trainer_time_forward(fv_trainer* tr, uint64_t step, uint32_t reps, double* seconds_per_launch);

/* Multi-GPU: one process per GPU.  Rank 0 draws an id, the caller ships the 128
 * bytes to the other ranks by any means, every rank calls init_comm.  Replaces
 * the reference's single-process peer access over managed memory
 * (cu_special_reduction.cu:61-66, 345-346). */
int fv_comm_unique_id(uint8_t id[128]);
int fv_trainer_init_comm(fv_trainer* tr, const uint8_t id[128]);
/* String-keyed tuning knobs in the manner of set_model_param_int / set_model_param_float
 * (model_descriptor.cu:50-112); none changes a result.
 *   "spin_limit"   polls a device-side wait for a peer's word makes before it gives up and the call
 *                  returns FV_ERR_TIMEOUT (default 8388608, about ten seconds);
 *   "tag_variant"  the scatter bookkeeping of a step: 1: one slot per thread and block round; 2: 1024 slots
 *                  deduplicated in shared memory before they are claimed; 3: several slots per thread, their
 *                  loads and claims issued together; 0 (default): 1 while a step fits the resident threads, else
 *                  3, or 2 where hot pairs are off or not every rank's windows are counted (see "hot_pairs");
 *   "tag_slots"    the slots per thread of the default variant: 1, 2, 4, 8, or 0 for the size-based choice;
 *   "colmax_lists" 1 (default): the largest untouched weight of every unit comes from a short list of
 *                  candidate rows kept from step to step (a unit whose list cannot certify its maximum
 *                  has its column read on the spot); 0: the matrix is streamed in every step (FV_COLMAX=scan
 *                  in the environment selects the same);
 *   "fused_update" 1 (default): in ordinary steps the evaluation of the normaliser and the update of the
 *                  touched weights run as one kernel whose CTAs meet once at a counter; 0: two kernels
 *                  (FV_FUSED_UPDATE=0 in the environment selects the same);
 *   "hot_pairs"    1 (default): requests for a (row of one of the 32 most frequent tokens, unit) pair are counted
 *                  by the forward pass and claimed once per pair by the tagging kernel, instead of queueing one by
 *                  one at the pair's address; ranks with peer mailboxes send one another their counts, ranks
 *                  that exchange through NCCL count their own windows only; 0: every request claims for itself
 *                  (FV_HOT_PAIRS=0 in the environment selects the same);
 *   "shard"        1 / 0: sharded or replicated update (peer mailboxes only; see fv_trainer_comm_mode);
 *   "loopback_peers" 1: test aid -- every peer's mailbox is mapped onto this rank's own, so a peer's
 *                  words never arrive and the first wait for one runs into spin_limit. */
int fv_trainer_set_option(fv_trainer* tr, const char* key, double value);
/* Multi-GPU from ONE process, as the reference drives its GPUs (train_flyvec.py:141-146: one
 * descriptor/arrays pair per device; cuda_funcs.cu:1664-1665: one OpenMP thread per GPU and step).
 * trs[r] must be rank r of world n.  With one device per rank the ranks map one another's mailboxes
 * through CUDA peer access and fv_trainers_run_* starts one host thread per GPU.  All ranks on ONE
 * device (for tests on a single GPU) share a stream and are advanced phase by phase, rank after rank,
 * so that a kernel never has to wait for one that has not run yet.  Every rank needs the corpus, the
 * weights and the window order set as for a single trainer.  nc_out / scale_out / stats may be NULL;
 * stats has n entries. */
int fv_trainers_link(fv_trainer* const* trs, int32_t n);
int fv_trainers_run_steps(fv_trainer* const* trs, int32_t n, uint64_t first_step, uint64_t nsteps, uint64_t warmup, float eps,
                          float* nc_out, float* scale_out, fv_run_stats* stats);
int fv_trainers_run_epoch(fv_trainer* const* trs, int32_t n, uint64_t epoch, uint64_t nep, fv_run_stats* stats);
/* winners[world*batch] and xx[world][K] of the last step as THIS rank received them (parity checks). */
int fv_trainer_last_packets(fv_trainer* tr, int32_t* winners, float* xx);
/* Counters of a trainer since its creation: "matrix_scans" = steps whose column maxima needed passes
 * over the whole synapse matrix (every step without candidate lists; with them only the step after new
 * weights or a fold); "column_rescans" = single units whose column had to be read in a step because all
 * their candidate rows had been touched. */
int fv_trainer_get_counter(fv_trainer* tr, const char* key, uint64_t* value);
/* How the ranks exchange their per-step packets (B winners and K floats of xx per rank):
 *   0  single rank / not initialised;
 *   1  one NCCL all-gather per step;
 *   2  peer-memory mailboxes: every packet word carries the step's sequence number beside its payload
 *      and is written with one 8-byte store straight into every peer's memory over NVLink, so no
 *      fence, flag or collective sits between the forward pass and the update; a consumer that finds
 *      an old sequence number polls that word, every poll loop is bounded, and a peer that never
 *      delivers ends the call with FV_ERR_TIMEOUT.
 * Mode 2 is chosen when every rank can map every other rank's mailbox; the environment variable
 * FV_COMM=nccl forces mode 1.  In mode 2 the update is replicated by default (every rank rebuilds every
 * rank's scatter from the exchanged winners: one exchange per step) or, with the "shard" option /
 * FV_SHARD=1 and delta == 0, sharded: rank r does the scatter bookkeeping and the column maxima for the
 * matrix rows i % world == r only and stores the count of every touched position into its peers' inboxes,
 * from which every replica applies the same update to its own copy (two exchanges per step, 1/world of
 * the bookkeeping). */
int fv_trainer_comm_mode(fv_trainer* tr, int* mode);
/* Which windows of the current order rank `rank` owns in global step `step`
 * (cuda_funcs.cu:1667-1670); pure arithmetic, usable without a GPU. */
int fv_shard_range(uint64_t num_windows, uint32_t batch, int32_t world, int32_t rank, uint64_t step,
                   uint64_t* first, uint64_t* count);

/* ---- hasher --------------------------------------------------------------
 * FlyVec.synapses / normalize_synapses (flyvec/core.py:22-36, 82-88): w_kn is the
 * checkpoint, float32 [K][N]; normalize != 0 divides each row by its 2-norm + prec.
 */
int fv_hasher_create(const float* w_kn, uint32_t hid, uint32_t n_cols, int normalize, float prec, int device,
                     fv_hasher** out);
int fv_hasher_destroy(fv_hasher* h);
/* The (possibly normalised) matrix back in checkpoint layout. */
int fv_hasher_get_weights(fv_hasher* h, float* w_kn);
/* FlyVec.get_sparse_embedding (flyvec/core.py:139-163) for a batch of token ids:
 * activations = column V+id, code = activation > midpoint of the hash_length-th
 * and next largest; id 0 gives zeros. */
int fv_hash_tokens(fv_hasher* h, const int32_t* ids, uint64_t n, uint32_t hash_length, uint32_t flags, uint8_t* out);
/* No counterpart in the reference.  Same result as fv_hash_tokens, but the call allocates nothing: ids and codes
 * are staged in a fixed 8 MiB device array that is part of the library (held by every GPU that loads it).  Meant for
 * callers that must not allocate while they hash: processes whose device memory belongs to another pool, or small
 * requests served next to a trainer that fills the GPU (fv_hash_tokens makes staging buffers on its first call).  n * (4 + bytes per code) + 256 must
 * fit into 8 MiB, else FV_ERR_INVALID.  The first call on a device looks up the array's address and should be made
 * before any stream capture is started; overlapping calls on one GPU race on the array. */
int fv_hash_tokens_static(fv_hasher* h, const int32_t* ids, uint64_t n, uint32_t hash_length, uint32_t flags,
                          uint8_t* out);
/* Context-dependent codes: activation of a window as the trainer's forward pass
 * computes it (cuda_funcs.cu:289-305 weighted by inv_freq, or 248-263 with
 * FV_HASH_RAW / inv_freq == NULL), then the same threshold rule. */
int fv_hash_windows(fv_hasher* h, const int32_t* idx, uint64_t nwin, uint32_t window, const float* inv_freq,
                    uint32_t hash_length, uint32_t flags, uint8_t* out);
/* Device-resident forms of the two calls above (ids / idx / out are device
 * pointers obtained from fv_device_alloc); they return when the kernel is done
 * and report its duration. */
int fv_hash_tokens_device(fv_hasher* h, const int32_t* d_ids, uint64_t n, uint32_t hash_length, uint32_t flags,
                          uint8_t* d_out, double* kernel_seconds);
int fv_hash_windows_device(fv_hasher* h, const int32_t* d_idx, uint64_t nwin, uint32_t window, int weighted,
                           uint32_t hash_length, uint32_t flags, uint8_t* d_out, double* kernel_seconds);
int fv_hasher_set_inverse_frequency(fv_hasher* h, const float* inv_freq, uint32_t vocab);

/* ---- raw buffers (cuda_helpers.cu:8-29 do_gpu_cudaHostAlloc & co.) ------- */
int fv_device_alloc(int device, size_t bytes, void** ptr);
int fv_device_free(int device, void* ptr);
int fv_host_alloc_pinned(size_t bytes, void** ptr);
int fv_host_free_pinned(void* ptr);
/* Free and total device memory as the CUDA runtime reports them (cudaMemGetInfo). */
int fv_device_mem_info(int device, size_t* free_bytes, size_t* total_bytes);
int fv_copy_to_device(int device, void* dst, const void* src, size_t bytes);
int fv_copy_to_host(int device, void* dst, const void* src, size_t bytes);
/* Writes `bytes` of a scratch buffer so that earlier data leave the L2 cache. */
int fv_flush_l2(int device, size_t bytes);

/* Measurement aid (no reference counterpart): read bandwidth of this GPU, measured on the spot, for the
 * two access patterns of the train step -- pattern 0: streaming 128-bit loads over `footprint` bytes;
 * pattern 1: whole rows of `row_bytes` gathered at random places, a warp per row -- each `reps` passes
 * after a warm-up pass.  A footprint that fits the L2 gives the L2's rate, a much larger one the HBM's. */
int fv_probe_read_bandwidth(int device, int pattern, size_t footprint, uint32_t row_bytes, uint32_t reps,
                            double* gbytes_per_s);

#ifdef __cplusplus
}
#endif
#endif /* FLYVEC_B200_H */
