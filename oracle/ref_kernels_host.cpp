// The reference's OWN training kernels, executed on the host -- TEST INFRASTRUCTURE ONLY.
//
// `ref_kernels.inc` is generated at build time by oracle/build_oracle.py: it holds the
// unmodified text of the reference's `__global__` functions, cut out of
// flyvec/src/cuda_funcs.cu and flyvec/src/cu_special_reduction.cu where they lie in a
// reference checkout (the generated file and the library built from it stay in the
// git-ignored oracle/_ref/).  cuda_on_host.h gives those functions CUDA's execution model
// on the CPU (blocks in order, threads of a block as lock-step fibers, the shuffle tree as
// the hardware performs it).  This file only restates the HOST side of one global step:
// which kernel is launched with which grid, block and arguments, in which order
//   per device   flyvec/src/cuda_funcs.cu:1664-1742   (run_epoch<int,int,1>, sparse input,
//                                                       frequency scaling, Lmid = Lbase = 1)
//   combine      flyvec/src/cu_special_reduction.cu:241-265
//   step size    flyvec/src/cuda_funcs.cu:1797-1799
//   update       flyvec/src/cu_special_reduction.cu:373-386
// so that the numpy and C restatements of the oracle can be checked, stage by stage,
// against arithmetic the reference's own source text performs.
//
// Two buffers are sized differently from the reference, on purpose:
//   * max_per_block holds 128*hid floats (what the kernel writes).  The reference allocates
//     ceil(hid*N/256) floats (cuda_funcs.cu:1531-1533, 1565), which is too small whenever
//     N < 32768;
//   * the finish kernel runs 512 threads on dynamic shared memory sized for 128
//     (cu_special_reduction.cu:243-252: 16 partial maxima written into room for 4 floats plus
//     the ngpus+1 counters); the host model's shared array is large enough to take them.
// Neither changes a value the step computes.
#include "cuda_on_host.h"

#include <vector>

#include "ref_kernels.inc"

namespace {

template <typename T>
std::vector<T*> row_table(T* base, size_t rows, size_t cols) {
  std::vector<T*> t(rows);
  for (size_t r = 0; r < rows; ++r) t[r] = base + r * cols;
  return t;
}

}  // namespace

extern "C" {

// One global step over `ngpus` replicas, all holding `model_in`.
//   tokens, ptr_offsets   the corpus and its window starts (model_arrays.cu:371-378 builds the same
//                         pointer table M1[i] = &tokens[ptr_offsets[i]])
//   myvector              window order; entries [g*Num, (g+1)*Num) are device g's windows of this step
// Outputs (any may be NULL): input ids [ngpus][Num][W], weighted and raw activations [ngpus][Num][hid],
// max_IDs [ngpus][Num][2], xx [ngpus][hid], the combined direction D [hid][N] (each device's chunk of
// columns, as left in its own ds), the updated model [hid][N] of replica 0, nc, the step size, and
// whether all replicas ended identical.
int refk_train_step(int hid, int N, int vocabulary_size, int W, int Num, int ngpus, int m, const float* model_in,
                    const int32_t* tokens, const uint64_t* ptr_offsets, uint64_t Ns_1, const uint64_t* myvector,
                    const float* word_inv_frequency, float eps, float delta, float prec, int32_t* input_out,
                    float* tot_input_out, float* tot_input_raw_out, int32_t* max_ids_out, float* xx_out, float* D_out,
                    float* model_out, float* nc_out, float* scale_out, int* replicas_identical) {
  if (hid < 1 || N < 1 || W < 1 || Num < 1 || ngpus < 1 || m < 1) return 1;
  const size_t KN = (size_t)hid * N;
  // per-device buffers (model_arrays.h:12-24)
  std::vector<std::vector<float>> syn(ngpus), dsv(ngpus), tot(ngpus), tot_raw(ngpus), xxv(ngpus), mpb(ngpus);
  std::vector<std::vector<int>> inp(ngpus), mids(ngpus);
  std::vector<std::vector<float*>> syn_t(ngpus), ds_t(ngpus), tot_t(ngpus), tot_raw_t(ngpus);
  std::vector<std::vector<int*>> inp_t(ngpus), mids_t(ngpus);
  std::vector<int*> M1(Ns_1);
  for (uint64_t i = 0; i < Ns_1; ++i) M1[i] = const_cast<int*>(tokens) + ptr_offsets[i];
  std::vector<float> freq(word_inv_frequency, word_inv_frequency + vocabulary_size);
  for (int g = 0; g < ngpus; ++g) {
    syn[g].assign(model_in, model_in + KN);
    dsv[g].assign(KN, 0.f);
    tot[g].assign((size_t)Num * hid, 0.f);
    tot_raw[g].assign((size_t)Num * hid, 0.f);
    xxv[g].assign(hid, 0.f);
    inp[g].assign((size_t)Num * W, -1);
    mids[g].assign((size_t)Num * 2, 0);
    mpb[g].assign((size_t)128 * hid, 0.f);
    syn_t[g] = row_table(syn[g].data(), hid, N);
    ds_t[g] = row_table(dsv[g].data(), hid, N);
    tot_t[g] = row_table(tot[g].data(), Num, hid);
    tot_raw_t[g] = row_table(tot_raw[g].data(), Num, hid);
    inp_t[g] = row_table(inp[g].data(), Num, W);
    mids_t[g] = row_table(mids[g].data(), Num, 2);
  }

  // launch geometry of run_epoch (cuda_funcs.cu:1521-1556)
  const size_t cuda_func_nthreads = 256;
  size_t cuda_func_nblocks = (KN + cuda_func_nthreads - 1) / cuda_func_nthreads;
  if (cuda_func_nblocks > 64 * 1024) cuda_func_nblocks = 64 * 1024;
  const int p_1 = 1;  // p = 2 (model_descriptor.cu:24-40; not settable from the driver)
  const int smem_max = 64 * (sizeof(int) + sizeof(float)) + m * (sizeof(int) + sizeof(float));
  int nthreads_scatter = 128;
  if (N < 33) nthreads_scatter = 32;
  else if (N < 65) nthreads_scatter = 64;
  else if (N < 97) nthreads_scatter = 96;
  const uint64_t IM_WIDTH = (uint64_t)W;  // unused by the kernel

  for (int g = 0; g < ngpus; ++g) {
    uint64_t* order = const_cast<uint64_t*>(myvector) + (size_t)g * Num;
    int** input = inp_t[g].data();
    float** ds = ds_t[g].data();
    float** synapses = syn_t[g].data();
    float** tot_input = tot_t[g].data();
    float** tot_input_raw = tot_raw_t[g].data();
    float* xx = xxv[g].data();
    int** max_IDs = mids_t[g].data();
    float* f = freq.data();
    int** m1 = M1.data();
    // cuda_funcs.cu:1679
    coh::launch(dim3(Num, 1, 1), dim3(32), 0,
                [&] { inflate_from_M_kernel_4<int>((uint64_t)Num, W, IM_WIDTH, (uint64_t)vocabulary_size, m1, order, input); }, false);
    // :1685-1688
    coh::launch(dim3((unsigned)cuda_func_nblocks), dim3((unsigned)cuda_func_nthreads), 0,
                [&] { cuda_func1_odd(hid * N, synapses[0], ds[0], p_1); }, false);
    // :1700-1701
    coh::launch(dim3(Num), dim3(32), 0,
                [&] { dense_sparse_matmul_special((uint64_t)Num, (uint64_t)hid, (uint64_t)N, W, ds, input, tot_input, f, vocabulary_size); },
                false);
    coh::launch(dim3(Num), dim3(32), 0,
                [&] { dense_sparse_matmul_special((uint64_t)Num, (uint64_t)hid, (uint64_t)N, W, ds, input, tot_input_raw); }, false);
    // :1715
    coh::launch(dim3((unsigned)cuda_func_nblocks), dim3((unsigned)cuda_func_nthreads), 0, [&] { fill_func_kernel(hid, xx, 0.0); }, false);
    // :1719 (the raw activations select)
    coh::launch(dim3(Num), dim3(64), smem_max, [&] { get_max_and_m_max_kernel_2(Num, hid, tot_input_raw, m, max_IDs); }, true);
    // :1721-1722
    coh::launch(dim3(Num), dim3(1), 0, [&] { xx_atomic_update_kernel(Num, max_IDs, xx, tot_input, delta); }, false);
    coh::launch(dim3(hid), dim3(N < 512 ? N : 512), 0, [&] { cuda_ds_xx_t_synapses_kernel(N, hid, ds, xx, synapses); }, false);
    // :1732
    coh::launch(dim3(Num), dim3(nthreads_scatter), 0,
                [&] { func_ds_eq_ds_input_kernel_sparse(Num, N, ds, W, input, max_IDs, delta, f, vocabulary_size); }, false);
  }

  // the combine (cu_special_reduction.cu:241-265), columns split by split_to_chuncks (cuda_funcs.cu:1658)
  std::vector<unsigned long long> offsets2D(ngpus + 1, 0ull);
  split_to_chuncks<float>((unsigned long long)N, (unsigned long long)ngpus, offsets2D.data());
  std::vector<float**> data2D(ngpus), model2D(ngpus);
  std::vector<float*> xx2D(ngpus);
  std::vector<int> device_list(ngpus);
  for (int g = 0; g < ngpus; ++g) {
    data2D[g] = ds_t[g].data();
    model2D[g] = syn_t[g].data();
    xx2D[g] = xxv[g].data();
    device_list[g] = g;
  }
  std::vector<float> max_abs_val(ngpus, 0.f);
  {
    const size_t nthreads = 128;
    const size_t smem = nthreads / 32 * sizeof(float) + sizeof(int) * (ngpus + 1);
    for (int dev = 0; dev < ngpus; ++dev) {
      float* mp = mpb[dev].data();
      float* out = &max_abs_val[dev];
      coh::launch(dim3(128, (unsigned)hid, 1), dim3((unsigned)nthreads), smem, [&] {
        reduce_by_chunks_and_absmax_kernel_sparse_2D<float>(data2D.data(), (uint64_t)hid, xx2D.data(), offsets2D.data(), device_list.data(),
                                                            ngpus, dev, mp);
      }, true);
      coh::launch(dim3(1), dim3(512), smem, [&] { max_of_AbsVal_kernel_finish<float>((size_t)128 * hid, mp, out); }, true);
    }
  }
  float nc = 0.0;
  for (int dev = 0; dev < ngpus; ++dev) nc = nc > max_abs_val[dev] ? nc : max_abs_val[dev];
  // cuda_funcs.cu:1797-1799
  float eps_inv_nc;
  if (prec > nc) eps_inv_nc = eps / prec;
  else eps_inv_nc = eps / nc;
  if (D_out) {
    for (int dev = 0; dev < ngpus; ++dev)
      for (int h = 0; h < hid; ++h)
        for (unsigned long long i = offsets2D[dev]; i < offsets2D[dev + 1]; ++i) D_out[(size_t)h * N + i] = ds_t[dev][h][i];
  }
  // the update (cu_special_reduction.cu:373-386)
  for (int dev = 0; dev < ngpus; ++dev) {
    float** data = data2D[dev];
    coh::launch(dim3(64, (unsigned)hid, 1), dim3(256), 0, [&] {
      update_model_multiGPU_kernel_sparse_2D<float>(data, offsets2D.data(), (uint64_t)hid, xx2D.data(), device_list.data(), ngpus,
                                                    model2D.data(), eps_inv_nc, dev);
    }, true);
  }

  int same = 1;
  for (int g = 1; g < ngpus; ++g) same &= (memcmp(syn[0].data(), syn[g].data(), KN * sizeof(float)) == 0);
  if (replicas_identical) *replicas_identical = same;
  for (int g = 0; g < ngpus; ++g) {
    if (input_out) memcpy(input_out + (size_t)g * Num * W, inp[g].data(), (size_t)Num * W * sizeof(int32_t));
    if (tot_input_out) memcpy(tot_input_out + (size_t)g * Num * hid, tot[g].data(), (size_t)Num * hid * sizeof(float));
    if (tot_input_raw_out) memcpy(tot_input_raw_out + (size_t)g * Num * hid, tot_raw[g].data(), (size_t)Num * hid * sizeof(float));
    if (max_ids_out) memcpy(max_ids_out + (size_t)g * Num * 2, mids[g].data(), (size_t)Num * 2 * sizeof(int32_t));
    if (xx_out) memcpy(xx_out + (size_t)g * hid, xxv[g].data(), (size_t)hid * sizeof(float));
  }
  if (model_out) memcpy(model_out, syn[0].data(), KN * sizeof(float));
  if (nc_out) *nc_out = nc;
  if (scale_out) *scale_out = eps_inv_nc;
  return 0;
}

// The winner search alone (cuda_funcs.cu:488-561 launched as at :1719) on caller-supplied activations
// [Num][hid]; max_ids [Num][2] = {winner, m-th winner}.  The activations are restored by the kernel itself.
int refk_get_max(int Num, int hid, int m, float* tot_input, int32_t* max_ids) {
  std::vector<float*> rows = row_table(tot_input, Num, hid);
  std::vector<int*> ids = row_table(max_ids, Num, 2);
  const int smem_max = 64 * (sizeof(int) + sizeof(float)) + m * (sizeof(int) + sizeof(float));
  float** t = rows.data();
  int** o = ids.data();
  coh::launch(dim3(Num), dim3(64), smem_max, [&] { get_max_and_m_max_kernel_2(Num, hid, t, m, o); }, true);
  return 0;
}

}  // extern "C"
