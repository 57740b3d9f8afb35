/* Weight-gradient GEMM on tcgen05 tensor cores, optionally fused with the cross-GPU
 * reduction of the result.
 *
 *   dW[M,N] (fp32, row-major) = dY[K,M]^T * X[K,N]      dY, X bf16 row-major
 *
 * Plain call (fused == NULL or nranks <= 1): dW may be any 16-byte aligned device buffer.
 *
 * Fused call: every rank calls with the same shapes. `dw` must be this rank's address of
 * a buffer that lives at the same offset of a symmetric, multicast-bound region on every
 * rank, `out_mc` the multicast address of the same buffer. As soon as a 128x256 tile has
 * been stored by all ranks, its owner (tile index mod nranks) lets the NVSwitch sum the
 * ranks' copies (multimem.ld_reduce.add.f32) and broadcasts the sum into every rank's
 * buffer (multimem.st) while the tensor cores continue with later tiles; the kernel returns
 * after a closing barrier, with the reduced (and scaled) gradient in every rank's dW.
 * This is the role the reference gives to "aggregate the gradient right where it is
 * produced"; the reference itself has no GPU code (its integrations copy gradients to host
 * memory first, frameworks_integration/pytorch_plugin/ProcessGroupSML.cpp:117-163).
 *
 * `flags_peer[r]` is rank r's copy of a flag array of switchml_wgrad_flag_words(M, N)
 * 64-bit words in symmetric memory, zero-initialised once; `epoch` must grow with every
* fused call that uses the same flag array, and `work_counter` must be zero when the kernel
 * starts. Waits give up after `timeout_ns` and set
 * *error_flag (device or mapped host memory) to 1.
 *
 * M and N must be multiples of 8 and all base addresses 16-byte aligned (TMA).
 * Returns 0, or < 0: -1 bad argument, -2 alignment, -3 tensor map, -4 launch.
 */
#ifndef SWITCHML_WGRAD_GEMM_H_
#define SWITCHML_WGRAD_GEMM_H_

#ifdef __cplusplus
extern "C" {
#endif

typedef struct WgradFusedArgs {
  int rank;
  int nranks;
  unsigned long long* flags_peer[8];
  char* out_mc;
  unsigned long long epoch;
  unsigned long long timeout_ns;
  float scale; /* multiplied into the reduced gradient (1/nranks for the mean) */
  int* work_counter; /* one int in this rank's device memory, zeroed (in stream order) before every fused call */
  /* mode 0 (default): every rank multiplies its own operands and the switch adds the ranks' results.
   * mode 1, "gather": the sum over ranks of dY_r^T X_r is ONE product over the concatenated K
   * dimension. Every rank first copies its dY and X into slab `rank` of a gather buffer on all
   * ranks (multimem.st; (nranks-1) * K * (M+N) * 2 bytes leave each GPU), then computes only the
   * tiles it owns (tile index mod nranks == rank) over all nranks * K rows and broadcasts them
   * (multimem.st) while the tensor cores go on. The link carries the gradient once instead of
   * (1 + 1/n) times in each direction plus the switch's reduction: the better plan whenever
   * the operands are small next to the gradient (VGG's fully connected layers: K = batch).
   * `gather_local` / `gather_mc`: this rank's and the multicast address of a buffer of
   * nranks * K * (M + N) bf16 in the symmetric region (same offset on every rank), laid out as
   * [nranks * K, M] followed by [nranks * K, N]; `gather_counter`: one zero-initialised int in
   * this rank's device memory (the kernel leaves it zero). */
  int mode;
  char* gather_local;
  char* gather_mc;
  int* gather_counter;
} WgradFusedArgs;

int switchml_wgrad_gemm(const void* dy, const void* x, float* dw, int M, int N, int K,
                        const WgradFusedArgs* fused, int* error_flag, void* stream);
/* Same GEMM (no fused reduce) with pairs of CTAs sharing 256x256 tiles (tcgen05 cta_group::2). */
int switchml_wgrad_gemm_2cta(const void* dy, const void* x, float* dw, int M, int N, int K,
                             int* error_flag, void* stream);
int switchml_wgrad_flag_words(int M, int N);

#ifdef __cplusplus
}
#endif
#endif /* SWITCHML_WGRAD_GEMM_H_ */
