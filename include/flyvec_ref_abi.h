/*
 * The reference's own ctypes ABI, served by libflyvec_b200.so (flyvec_b200/csrc/fv_shim.cu).
 *
 * bhoov/flyvec's Python driver loads five shared objects and calls the functions below
 * (flyvec/train_flyvec.py:62-259).  libflyvec_b200.so exports all of them under the same names and
 * signatures, so the unmodified driver runs on this library when its five CDLL paths point at copies
 * or links of it (`flyvec_compile` creates them in flyvec_b200/csrc/ref_abi/).  One GPU only; window
 * order from a seeded shuffle (environment FLYVEC_SEED).  Citations: file:line in the reference.
 */
#ifndef FLYVEC_REF_ABI_H
#define FLYVEC_REF_ABI_H
#include <stdint.h>
#ifdef __cplusplus
extern "C" {
#endif

/* cuda_helpers.so -- flyvec/src/cuda_helpers.cu:8-35 */
void* do_gpu_cudaMallocManaged(unsigned long size);
void* do_cpu_malloc(unsigned long size);
void* do_gpu_cudaHostAlloc(unsigned long size);
int get_cuda_num_devices(void); /* answers 1: the shim drives one GPU */

/* prune_input.so -- flyvec/src/prune_input.cpp:13-122 */
void prune_input_data(void* DATA_in, uint64_t Nrows, uint64_t Ncolumns);
uint64_t getnum_samples(void* offsets_in, uint64_t Nsentences, uint64_t W);
void compute_offset_phrases(void* offset_phrases_in, void* offsets_sentences_in, uint64_t Nsentences, uint64_t W);

/* model_descriptor.so -- flyvec/src/model_descriptor.cu:17-180 */
void* model_create_descriptor(int num_gpus);
void set_model_param_int(uint64_t value, const char* s, void* MODEL);
void set_model_param_float(float value, const char* s, void* MODEL);
void compute_model_derived_parameters(void* MODEL);
void copy_model_params(void* MODEL, int from, int to);
void print_model_params(void* MODEL);

/* model_arrays.so -- flyvec/src/model_arrays.cu:14-448 */
void* model_create_arrays(int num_gpus);
void model_arrays_allocate_memory(void* descr_in, void* MA_in, int num_gpus);
void push_INPUT_memory_to_GPU(void* MA_in, void* descr_in, int deviceID, const char* type);
void* get_data_pointer(const char* s, void* MA_in, int deviceID); /* "synapses": float [hid][2V] host slab */
void set_data_pointer(const char* s, void* MA_in, void* descr_in, void* ptr, const char* type, int deviceID);
void set_up_INPUT_pointer(const char* s, void* MA_in, void* descr_in, void* ptr_in, void* ptr_offsets_in,
                          const char* type, int deviceID);
void compute_inverse_word_frequency(void* MA_in, void* descr_in, void* input_in, uint64_t Nwords, int deviceID);
void do_reshuffle_indices(void* descr_in, void* MA_in, int deviceID);

/* cuda_funcs.so -- flyvec/src/cuda_funcs.cu:1163-1257 */
void launch_epoch_INPUT_AS_INT(void* descr_in, void* MA_in, int num_gpus, uint64_t epoch_id, uint64_t Nep);
void launch_epoch_INPUT_AS_IMAGE(void* descr_in, void* MA_in, int num_gpus, uint64_t epoch_id, uint64_t Nep);
void launch_epoch_INPUT_AS_FLOAT(void* descr_in, void* MA_in, int num_gpus, uint64_t epoch_id, uint64_t Nep);

#ifdef __cplusplus
}
#endif
#endif /* FLYVEC_REF_ABI_H */
