// The reference's own ctypes ABI (24 extern "C" names spread over model_descriptor.so,
// model_arrays.so, cuda_helpers.so, cuda_funcs.so and prune_input.so, called from
// flyvec/train_flyvec.py:62-259) implemented on top of the fv_* entry points, so that the
// reference's unmodified Python driver can run on this library: point its five CDLL loads at
// copies (or links) of libflyvec_b200.so.
//
// Same names, argument order and meaning; like the reference the functions return nothing and
// report problems on stderr.  The shim drives ONE GPU (get_cuda_num_devices answers 1); the
// multi-GPU path is one process per GPU and goes through flyvec_b200's own driver.
// Differences a caller can observe: the window order comes from fv_trainer_shuffle (seeded from
// the environment variable FLYVEC_SEED, default 0) instead of the reference's quasi-random
// transposition shuffle; "synapses" is a pinned host slab that is uploaded at the start of every
// launch_epoch_INPUT_AS_INT and refreshed at its end (the reference hands out managed memory).
#include <cstdio>
#include <cstdlib>
#include <cstring>

#include "fv_common.h"

namespace {

struct ShimDescr {  // model_descriptor.h:13-66, the fields the driver sets
  uint64_t IM_HEIGHT = 32, IM_WIDTH = 32, Nchannels = 3, Ns_1 = 0, W = 4, ST = 1, hid = 100, Num = 100, m = 2, p = 2;
  uint64_t vocabulary_size = 0, sparse_input = 0, frequency_scaling = 0;
  float initial_learning_rate = 0.001f, delta = 0.f, prec = 1.0e-30f, mu = 0.f, sigma = 1.f, Lmid = 1.f, Lbase = 1.f;
  int count = 1;
};

struct ShimArrays {  // what model_arrays holds for the driver
  fv_trainer* tr = nullptr;
  float* slab = nullptr;  // "synapses": pinned host memory, float [hid][2V]
  const int32_t* input = nullptr;
  const uint64_t* starts = nullptr;
  bool corpus_set = false;
  uint64_t shuffles = 0;
  int count = 1;
};

void complain(const char* where) { fprintf(stderr, "%s: %s\n", where, fv_last_error()); }

}  // namespace

extern "C" {

// ---- cuda_helpers.cu:8-35 ----------------------------------------------------------------
void* do_gpu_cudaMallocManaged(unsigned long size) {
  void* p = nullptr;
  if (cudaMallocManaged(&p, size) != cudaSuccess) return nullptr;
  return p;
}
void* do_cpu_malloc(unsigned long size) { return malloc(size); }
void* do_gpu_cudaHostAlloc(unsigned long size) {
  void* p = nullptr;
  if (fv_host_alloc_pinned(size, &p) != FV_OK) {
    complain("do_gpu_cudaHostAlloc");
    return nullptr;
  }
  return p;
}
int get_cuda_num_devices() {
  int n = 0;
  if (fv_device_count(&n) != FV_OK || n < 1) return 0;
  return 1;  // the shim drives one GPU
}

// ---- prune_input.cpp:13-122 --------------------------------------------------------------
uint64_t getnum_samples(void* offsets_in, uint64_t Nsentences, uint64_t W) {
  uint64_t n = 0;
  if (fv_enumerate_windows((const uint64_t*)offsets_in, Nsentences, (uint32_t)W, 0, &n, nullptr) != FV_OK)
    complain("getnum_samples");
  fprintf(stderr, "%lu phrases with W %ld  words\n", (unsigned long)n, (long)W);
  return n;
}
void compute_offset_phrases(void* offset_phrases_in, void* offsets_sentences_in, uint64_t Nsentences, uint64_t W) {
  uint64_t n = 0;
  if (fv_enumerate_windows((const uint64_t*)offsets_sentences_in, Nsentences, (uint32_t)W, 0, &n,
                           (uint64_t*)offset_phrases_in) != FV_OK)
    complain("compute_offset_phrases");
}
// De-duplication of window entries; the reference exports it but its driver never calls it.
void prune_input_data(void* DATA_in, uint64_t Nrows, uint64_t Ncolumns) {
  int* data = (int*)DATA_in;
  const uint64_t mid = Ncolumns / 2;
  for (uint64_t row = 0; row < Nrows; ++row) {
    int* r = data + row * Ncolumns;
    for (uint64_t c = 1; c < Ncolumns; ++c) {
      if (c == mid) continue;
      for (uint64_t cc = 0; cc < c; ++cc)
        if (cc != mid && r[cc] == r[c]) {
          r[c] = -1;
          break;
        }
    }
  }
}

// ---- model_descriptor.cu:17-180 ----------------------------------------------------------
void* model_create_descriptor(int num_gpus) {
  if (num_gpus < 1) num_gpus = 1;
  ShimDescr* d = new ShimDescr[num_gpus];
  for (int g = 0; g < num_gpus; ++g) d[g].count = num_gpus;
  return d;
}
void set_model_param_int(uint64_t value, const char* s, void* MODEL) {
  ShimDescr* M = (ShimDescr*)MODEL;
  if (!strcmp(s, "IM_HEIGHT")) M->IM_HEIGHT = value;
  else if (!strcmp(s, "IM_WIDTH")) M->IM_WIDTH = value;
  else if (!strcmp(s, "Nchannels")) M->Nchannels = value;
  else if (!strcmp(s, "Ns_1")) M->Ns_1 = value;
  else if (!strcmp(s, "W")) M->W = value;
  else if (!strcmp(s, "ST")) M->ST = value;
  else if (!strcmp(s, "hid")) M->hid = value;
  else if (!strcmp(s, "Num")) M->Num = value;
  else if (!strcmp(s, "p")) M->p = value;
  else if (!strcmp(s, "m")) M->m = value;
  else if (!strcmp(s, "vocabulary_size")) M->vocabulary_size = value;
  else if (!strcmp(s, "sparse_input")) M->sparse_input = value;
  else if (!strcmp(s, "frequency_scaling")) M->frequency_scaling = value;
  else printf("set_param_int: unknown parameter %s\n", s);
}
void set_model_param_float(float value, const char* s, void* MODEL) {
  ShimDescr* M = (ShimDescr*)MODEL;
  if (!strcmp(s, "initial_learning_rate")) M->initial_learning_rate = value;
  else if (!strcmp(s, "delta")) M->delta = value;
  else if (!strcmp(s, "prec")) M->prec = value;
  else if (!strcmp(s, "mu")) M->mu = value;
  else if (!strcmp(s, "sigma")) M->sigma = value;
  else if (!strcmp(s, "Lmid")) M->Lmid = value;
  else if (!strcmp(s, "Lbase")) M->Lbase = value;
  else printf("set_param_float: unknown parameter %s\n", s);
}
void compute_model_derived_parameters(void*) {}  // N = 2*vocabulary_size is implied; no cuRAND generator to create
void copy_model_params(void* MODEL, int from, int to) {
  ShimDescr* M = (ShimDescr*)MODEL;
  if (from >= 0 && to >= 0 && from < M->count && to < M->count) M[to] = M[from];
}
void print_model_params(void* MODEL) {
  const ShimDescr* M = (const ShimDescr*)MODEL;
  fprintf(stderr, "Ns_1=%lu W=%lu hid=%lu Num=%lu vocabulary_size=%lu lr=%g delta=%g prec=%g\n", (unsigned long)M->Ns_1,
          (unsigned long)M->W, (unsigned long)M->hid, (unsigned long)M->Num, (unsigned long)M->vocabulary_size,
          M->initial_learning_rate, M->delta, M->prec);
}

// ---- model_arrays.cu:14-448 --------------------------------------------------------------
void* model_create_arrays(int num_gpus) {
  if (num_gpus < 1) num_gpus = 1;
  ShimArrays* a = new ShimArrays[num_gpus];
  for (int g = 0; g < num_gpus; ++g) a[g].count = num_gpus;
  return a;
}
void model_arrays_allocate_memory(void* descr_in, void* MA_in, int /*num_gpus*/) {
  const ShimDescr* D = (const ShimDescr*)descr_in;
  ShimArrays* A = (ShimArrays*)MA_in;
  if (D->sparse_input == 0 || D->Lmid != 1.f || D->Lbase != 1.f)
    fprintf(stderr, "model_arrays_allocate_memory: only sparse_input = 1 with Lmid = Lbase = 1 is implemented\n");
  fv_config cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.struct_size = sizeof(cfg);
  cfg.device = 0;
  cfg.rank = 0;
  cfg.world = 1;
  cfg.hid = (uint32_t)D->hid;
  cfg.vocab = (uint32_t)D->vocabulary_size;
  cfg.window = (uint32_t)D->W;
  cfg.batch = (uint32_t)D->Num;
  cfg.lr0 = D->initial_learning_rate;
  cfg.delta = D->delta;
  cfg.prec = D->prec;
  cfg.m = (uint32_t)D->m;
  cfg.flags = FV_FLAG_COUNT_FP32;  // the reference counts words in a float (model_arrays.cu:413-416)
  if (fv_trainer_create(&cfg, &A->tr) != FV_OK) {
    complain("model_arrays_allocate_memory");
    return;
  }
  void* slab = nullptr;
  if (fv_host_alloc_pinned((size_t)D->hid * 2 * D->vocabulary_size * sizeof(float), &slab) != FV_OK) {
    complain("model_arrays_allocate_memory");
    return;
  }
  A->slab = (float*)slab;
  memset(A->slab, 0, (size_t)D->hid * 2 * D->vocabulary_size * sizeof(float));
}
void push_INPUT_memory_to_GPU(void*, void*, int, const char*) {}  // the corpus is uploaded by compute_inverse_word_frequency
void* get_data_pointer(const char* s, void* MA_in, int deviceID) {
  ShimArrays* A = (ShimArrays*)MA_in;
  if (!strcmp(s, "synapses") && deviceID == 0) return A->slab;
  return nullptr;
}
void set_data_pointer(const char* s, void*, void*, void*, const char*, int) {
  printf("set_data_pointer: %s is not used by the text trainer\n", s);
}
void set_up_INPUT_pointer(const char*, void* MA_in, void*, void* ptr_in, void* ptr_offsets_in, const char* type,
                          int deviceID) {
  ShimArrays* A = (ShimArrays*)MA_in;
  if (deviceID != 0) return;
  if (strcmp(type, "i4") && strcmp(type, "I4")) {
    printf("set_up_INPUT_pointer: only int32 token ids (\"i4\") are implemented\n");
    return;
  }
  A->input = (const int32_t*)ptr_in;
  A->starts = (const uint64_t*)ptr_offsets_in;
}
void compute_inverse_word_frequency(void* MA_in, void* descr_in, void* input_in, uint64_t Nwords, int deviceID) {
  ShimArrays* A = (ShimArrays*)MA_in;
  const ShimDescr* D = (const ShimDescr*)descr_in;
  if (deviceID != 0 || !A->tr) return;
  if (!A->starts) {
    fprintf(stderr, "compute_inverse_word_frequency: set_up_INPUT_pointer has not been called\n");
    return;
  }
  // the tokens, the window table and the counts reach the GPU here
  if (fv_trainer_set_corpus_windows(A->tr, (const int32_t*)input_in, Nwords, A->starts, D->Ns_1) != FV_OK) {
    complain("compute_inverse_word_frequency");
    return;
  }
  A->corpus_set = true;
}
void do_reshuffle_indices(void*, void* MA_in, int deviceID) {
  ShimArrays* A = (ShimArrays*)MA_in;
  if (deviceID != 0 || !A->tr || !A->corpus_set) return;
  const char* s = getenv("FLYVEC_SEED");
  const uint64_t base = s ? strtoull(s, nullptr, 10) : 0;
  if (fv_trainer_shuffle(A->tr, base * 1000003ull + A->shuffles) != FV_OK) complain("do_reshuffle_indices");
  A->shuffles += 1;
}

// ---- cuda_funcs.cu:1163-1257 -------------------------------------------------------------
void launch_epoch_INPUT_AS_INT(void* descr_in, void* MA_in, int /*num_gpus*/, uint64_t epoch_id, uint64_t Nep) {
  ShimArrays* A = (ShimArrays*)MA_in;
  (void)descr_in;
  if (!A->tr || !A->corpus_set) {
    fprintf(stderr, "launch_epoch_INPUT_AS_INT: the corpus has not been set up\n");
    return;
  }
  if (fv_trainer_set_weights(A->tr, A->slab) != FV_OK) return complain("launch_epoch_INPUT_AS_INT");
  fv_run_stats st;
  if (fv_trainer_run_epoch(A->tr, epoch_id, Nep, &st) != FV_OK) return complain("launch_epoch_INPUT_AS_INT");
  if (fv_trainer_get_weights(A->tr, A->slab) != FV_OK) return complain("launch_epoch_INPUT_AS_INT");
  fprintf(stderr, "  run_epoch: %llu steps, %.4g windows/s on the GPU\n", (unsigned long long)st.steps,
          st.seconds > 0 ? (double)st.windows / st.seconds : 0.0);
}
void launch_epoch_INPUT_AS_IMAGE(void*, void*, int, uint64_t, uint64_t) {
  fprintf(stderr, "launch_epoch_INPUT_AS_IMAGE: image inputs are not implemented\n");
}
void launch_epoch_INPUT_AS_FLOAT(void*, void*, int, uint64_t, uint64_t) {
  fprintf(stderr, "launch_epoch_INPUT_AS_FLOAT: dense float inputs are not implemented\n");
}

}  // extern "C"
