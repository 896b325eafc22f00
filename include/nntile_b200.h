/* nntile_b200 - B200 (sm_100a) kernels for NNTile's tiled scaled-dot-product
 * attention path, behind a plain C ABI.
 *
 * Conventions shared by every entry point (they are those of the reference's
 * nntile::kernel::<op>::cuda<T> functions, include/nntile/kernel/cuda.hh:85-120):
 *   - the first argument is the CUDA stream (a cudaStream_t passed as void*);
 *     work is only ENQUEUED on it, nothing synchronises;
 *   - sizes are int64_t (NNTile's Index), scalars are float (NNTile's Scalar);
 *   - all pointers are DEVICE pointers owned by the caller for the lifetime of
 *     the enqueued work; the library allocates nothing;
 *   - arrays are Fortran order (first index fastest), fp32 or bfloat16
 *     (bit-compatible with nntile::bf16_t / __nv_bfloat16); the fused pair also
 *     takes IEEE half (nntile::fp16_t / __half);
 *   - the return value is a status: 0 = enqueued, negative = rejected before any
 *     launch (see NNTILE_B200_E_*).  Nothing is thrown and nothing is printed.
 *
 * Every declaration cites the reference interface it replaces as file:line,
 * relative to the reference tree (nntile/nntile v1.1.0).
 */
#ifndef NNTILE_B200_H
#define NNTILE_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define NNTILE_B200_OK 0
#define NNTILE_B200_E_BADARG (-1)   /* null pointer, negative or inconsistent size */
#define NNTILE_B200_E_SHAPE (-2)    /* shape not supported by this entry point */
#define NNTILE_B200_E_ALIGN (-3)    /* pointer not aligned as documented */
#define NNTILE_B200_E_SCRATCH (-4)  /* caller-provided scratch/workspace too small */
#define NNTILE_B200_E_LAUNCH (-5)   /* CUDA refused the launch (cudaGetLastError) */
#define NNTILE_B200_E_DEVICE (-6)   /* device is not compute capability 10.x */

typedef void *nntile_b200_stream_t; /* cudaStream_t */

/* Library version (major*10000 + minor*100 + patch) and status text. */
int nntile_b200_version(void);
const char *nntile_b200_status_string(int status);
/* Number of CUDA kernels this library has launched in this process so far
 * (memsets are not kernels).  No reference counterpart: a measurement aid. */
unsigned long long nntile_b200_launch_count(void);

/* ---------------------------------------------------------------------------
 * Unfused chain (the "vanilla" path of nntile.layer.Sdpa)
 * ------------------------------------------------------------------------- */

/* if(!mask[i]) data[i,:] = val, data is nrows-by-ncols.
 * Replaces nntile::kernel::mask_scalar::cuda<T>,
 * include/nntile/kernel/mask_scalar/cuda.hh:25, src/kernel/mask_scalar/cuda.cu:21-110. */
int nntile_b200_mask_scalar_fp32(nntile_b200_stream_t stream, int64_t nrows,
        int64_t ncols, const uint8_t *mask, float val, float *data);
int nntile_b200_mask_scalar_bf16(nntile_b200_stream_t stream, int64_t nrows,
        int64_t ncols, const uint8_t *mask, float val, void *data);

/* Running (max, sum exp(x-max)) of every fibre src[i,:,j] of an m-by-k-by-n array,
 * merged into the interleaved 2-by-m-by-n `maxsumexp`; infinite entries are
 * ignored, a stored sum of zero means "empty".
 * Replaces nntile::kernel::maxsumexp::cuda<T>,
 * include/nntile/kernel/maxsumexp/cuda.hh:25, src/kernel/maxsumexp/cuda.cu:22-323. */
int nntile_b200_maxsumexp_fp32(nntile_b200_stream_t stream, int64_t m, int64_t n,
        int64_t k, const float *src, float *maxsumexp);
int nntile_b200_maxsumexp_bf16(nntile_b200_stream_t stream, int64_t m, int64_t n,
        int64_t k, const void *src, void *maxsumexp);

/* dst[i,l,j] = alpha*exp(dst[i,l,j]-max[i,j])/sum[i,j]; infinite entries -> 0.
 * Replaces nntile::kernel::softmax_inplace::cuda<T>,
 * include/nntile/kernel/softmax_inplace/cuda.hh:25, src/kernel/softmax_inplace/cuda.cu:22-181. */
int nntile_b200_softmax_inplace_fp32(nntile_b200_stream_t stream, int64_t m,
        int64_t n, int64_t k, const float *maxsumexp, float alpha, float *dst);
int nntile_b200_softmax_inplace_bf16(nntile_b200_stream_t stream, int64_t m,
        int64_t n, int64_t k, const void *maxsumexp, float alpha, void *dst);

/* dst[i,j] = beta*dst[i,j] + alpha*sum_l src1[i,l,j]*src2[i,l,j]; beta==0 does not
 * read dst.  Replaces nntile::kernel::sumprod_slice::cuda<T>,
 * include/nntile/kernel/sumprod_slice/cuda.hh:25, src/kernel/sumprod_slice/cuda.cu:22-214. */
int nntile_b200_sumprod_slice_fp32(nntile_b200_stream_t stream, int64_t m,
        int64_t n, int64_t k, float alpha, const float *src1, const float *src2,
        float beta, float *dst);
int nntile_b200_sumprod_slice_bf16(nntile_b200_stream_t stream, int64_t m,
        int64_t n, int64_t k, float alpha, const void *src1, const void *src2,
        float beta, void *dst);

/* dst[i,l,j] = beta*dst[i,l,j] + alpha*src[i,j].
 * Replaces nntile::kernel::add_slice_inplace::cuda<T>,
 * include/nntile/kernel/add_slice_inplace/cuda.hh:25, src/kernel/add_slice_inplace/cuda.cu:22-158. */
int nntile_b200_add_slice_inplace_fp32(nntile_b200_stream_t stream, int64_t m,
        int64_t n, int64_t k, float alpha, const float *src, float beta, float *dst);
int nntile_b200_add_slice_inplace_bf16(nntile_b200_stream_t stream, int64_t m,
        int64_t n, int64_t k, float alpha, const void *src, float beta, void *dst);

/* dst = alpha*src*dst.  Replaces nntile::kernel::multiply_inplace::cuda<T>,
 * include/nntile/kernel/multiply_inplace/cuda.hh:25, src/kernel/multiply_inplace/cuda.cu:21-76. */
int nntile_b200_multiply_inplace_fp32(nntile_b200_stream_t stream, int64_t nelems,
        float alpha, const float *src, float *dst);
int nntile_b200_multiply_inplace_bf16(nntile_b200_stream_t stream, int64_t nelems,
        float alpha, const void *src, void *dst);

/* dst = alpha*src + beta*dst.  Replaces nntile::kernel::add_inplace::cuda<T>,
 * include/nntile/kernel/add_inplace/cuda.hh:25. */
int nntile_b200_add_inplace_fp32(nntile_b200_stream_t stream, int64_t nelems,
        float alpha, const float *src, float beta, float *dst);
int nntile_b200_add_inplace_bf16(nntile_b200_stream_t stream, int64_t nelems,
        float alpha, const void *src, float beta, void *dst);

/* dst[i] = val (fp32) and dst bytes = 0: the prologue of the fused forward
 * (lse = -inf, A = 0; wrappers/python/nntile/layer/sdpa.py:538-539).
 * Replace nntile::kernel::fill::cuda<fp32_t>, include/nntile/kernel/fill/cuda.hh:24,
 * and the clear codelet, src/starpu/clear.cc. */
int nntile_b200_fill_fp32(nntile_b200_stream_t stream, int64_t nelems, float val,
        float *dst);
int nntile_b200_clear(nntile_b200_stream_t stream, int64_t nbytes, void *dst);

/* Merge a partial attention result (src_lse[seq*batch], src_attn[head, seq*batch])
 * into the running one by log-sum-exp weights; rows whose incoming lse is not
 * finite are left untouched.
 * Replaces nntile::kernel::accumulate_attn_output::cuda<T>,
 * include/nntile/kernel/accumulate_attn_output/cuda.hh:25,
 * src/kernel/accumulate_attn_output/cuda.cu:28-135. */
int nntile_b200_accumulate_attn_output_fp32(nntile_b200_stream_t stream,
        int64_t head, int64_t seq, int64_t batch, const float *src_lse,
        const float *src_attn, float *dst_lse, float *dst_attn);
int nntile_b200_accumulate_attn_output_bf16(nntile_b200_stream_t stream,
        int64_t head, int64_t seq, int64_t batch, const float *src_lse,
        const void *src_attn, float *dst_lse, void *dst_attn);

/* Batched column-major GEMM, C[m,n,batch] = alpha*op(A)*op(B) + beta*C with packed
 * leading dimensions and the matrices of a batch back to back; transA / transB are
 * 0 (as stored) or 1 (transposed); alpha and beta act on the fp32 accumulator before
 * the single rounding to the storage type.  `cublas_handle` is the caller's
 * cublasHandle_t, already bound to the stream the work should run on - in the
 * reference the StarPU worker's handle.  A library call in the reference and here
 * (cublasGemmStridedBatchedEx, fp32 compute, looked up in the process at run time;
 * NNTILE_B200_E_DEVICE if no cuBLAS can be found).
 * Replaces nntile::kernel::cublas::gemm<T>, include/nntile/kernel/cublas.hh,
 * src/kernel/cublas.cc:35-164 (same argument order). */
int nntile_b200_gemm_fp32(void *cublas_handle, int transA, int transB, int64_t m,
        int64_t n, int64_t k, int64_t batch, float alpha, const float *A, const float *B,
        float beta, float *C);
int nntile_b200_gemm_bf16(void *cublas_handle, int transA, int transB, int64_t m,
        int64_t n, int64_t k, int64_t batch, float alpha, const void *A, const void *B,
        float beta, void *C);

/* ---------------------------------------------------------------------------
 * Fused flash SDPA, one (Q tile, K/V tile) task
 * ------------------------------------------------------------------------- */

/* Forward: (lse, A) <- merge((lse, A), SDPA(Q, K, V, bias=mask, scale=1/sqrt(head))).
 * Per batch entry K, Q, V, A are row-major [seq][head] matrices, `batch` of them
 * back to back; mask is the additive bias [seq_q][seq_k] row major in bf16
 * (0 = keep, -inf = drop, any finite value allowed); lse is fp32 [batch][seq].
 * The caller initialises lse = -inf, A = 0 before the first K/V tile of a Q tile.
 * scratch_lse (seq*batch floats) and scratch_A (seq*head*batch bf16) are the two
 * scratch buffers the reference's tile layer hands to every task; they may be
 * overwritten with anything.  All pointers 16-byte aligned.
 * For shapes the tcgen05 kernels take, the first 4 bytes of scratch_A are the task's
 * status word (see nntile_b200_flash_sdpa_read_status).
 * Pointer order and semantics are those of
 * nntile::kernel::flash_sdpa_fwd_cudnn::execute_graph<bf16_t>,
 * include/nntile/kernel/flash_sdpa_fwd_cudnn/cuda.hh:37-76,
 * src/kernel/flash_sdpa_fwd_cudnn/cuda.cc:145-202 (cuDNN graph + merge), with the
 * cudnnHandle_t/graph pair replaced by the stream. */
int nntile_b200_flash_sdpa_fwd_bf16(nntile_b200_stream_t stream, int64_t seq,
        int64_t head, int64_t batch, const void *K, const void *Q,
        const void *mask, float *scratch_lse, const void *V, void *scratch_A,
        float *lse, void *A);

/* Backward: dK, dQ, dV += gradients of one (Q tile, K/V tile) pair computed from
 * the GIVEN A (final output) and lse (final log-sum-exp) of the Q tile.
 * The three scratch buffers (each seq*head*batch bf16) may be overwritten; for shapes
 * the tcgen05 kernels take, the first 4 bytes of scratch_dV are the task's status word.
 * Pointer order and semantics are those of
 * nntile::kernel::flash_sdpa_bwd_cudnn::execute_graph<bf16_t>,
 * include/nntile/kernel/flash_sdpa_bwd_cudnn/cuda.hh:29-59,
 * src/kernel/flash_sdpa_bwd_cudnn/cuda.cc:171-218; no separate workspace. */
int nntile_b200_flash_sdpa_bwd_bf16(nntile_b200_stream_t stream, int64_t seq,
        int64_t head, int64_t batch, const void *K, const void *Q, const void *V,
        const void *A, const void *dA, const void *mask, const float *lse,
        void *scratch_dK, void *scratch_dQ, void *scratch_dV, void *dK, void *dQ,
        void *dV);

/* Grouped-query form of the two tile tasks above: Q, A, dA, dQ are
 * [head, seq, batch, group, kv_heads], K, V, dK, dV are [head, seq, batch, kv_heads]
 * and are NOT replicated over the group.  The reference has no such entry point: its
 * attention layers replicate K and V `group` times before the SDPA layer and sum the
 * K/V gradients over the group afterwards (wrappers/python/nntile/model/
 * llama_attention.py:605-616, 786-793: add_slice_inplace forward, sum_slice
 * backward); calling these instead drops both passes and reads K/V once per kv
 * head.  Same mask, lse and merge / "+=" contracts as the entry points above; dK and
 * dV receive the sum over the group.  Only shapes the tcgen05 kernels take (head 64
 * or 128, seq a multiple of 128), NNTILE_B200_E_SHAPE otherwise.  `scratch` holds at
 * least nntile_b200_flash_sdpa_gqa_scratch_bytes(...) bytes for the backward and
 * 256 + (seq/128)^2 bytes for the forward, 16-byte aligned. */
int nntile_b200_flash_sdpa_fwd_gqa_bf16(nntile_b200_stream_t stream, int64_t seq,
        int64_t head, int64_t batch, int64_t group, int64_t kv_heads, const void *K,
        const void *Q, const void *mask, const void *V, float *lse, void *A,
        void *scratch, size_t scratch_bytes);
int nntile_b200_flash_sdpa_bwd_gqa_bf16(nntile_b200_stream_t stream, int64_t seq,
        int64_t head, int64_t batch, int64_t group, int64_t kv_heads, const void *K,
        const void *Q, const void *V, const void *A, const void *dA, const void *mask,
        const float *lse, void *dK, void *dQ, void *dV, void *scratch,
        size_t scratch_bytes);
size_t nntile_b200_flash_sdpa_gqa_scratch_bytes(int64_t seq, int64_t head,
        int64_t batch, int64_t group, int64_t kv_heads);

/* Status word of the tcgen05 kernels.  Every wait inside them is bounded; a role
 * that gives up (a copy or a product it waits for did not arrive within 200 ms)
 * stores a code in a 32-bit word in device memory, the CTAs of the launch - and of
 * every later launch that shares the word - skip their work, and the kernels return
 * normally: the C call has long returned NNTILE_B200_OK by then, and the outputs of
 * the skipped CTAs are NOT valid.  The word is the first 4 bytes of the buffer that
 * carries the task's bookkeeping: scratch_A (forward tile task), scratch_dV (backward
 * tile task), `scratch` (grouped-query and tensor-level entry points).  A tile-level
 * call clears it when it starts; a tensor-level call clears it once and every one of
 * its tasks shares it, so a give-up in any task stays visible (and stops the tasks
 * behind it).  Codes: 0 clean; forward 1 producer, 2 MMA issuer, 3 softmax; backward
 * 11 producer, 12 MMA issuer, 13 dQ drain, 14 softmax, 20 shared memory misaligned.
 * This helper copies the word to the host: it SYNCHRONISES `stream` (the one call of
 * this library that does) and is meant for after a step, not between tasks.
 * No counterpart in the reference (cuDNN reports through its own status). */
int nntile_b200_flash_sdpa_read_status(nntile_b200_stream_t stream, const void *scratch,
        unsigned int *code);

/* Test support, no counterpart in the reference: arms a one-shot hook for the NEXT
 * tcgen05 forward launch of this process.  That launch runs a test instantiation of
 * the kernel whose waits give up after 1 ms and whose producer withholds the first K
 * copy, so that one wait runs out, the status word becomes non-zero and the kernel
 * returns normally.  Nothing traps or spins; used by the test of the failure report. */
void nntile_b200_test_arm_wait_timeout(void);

/* IEEE half (nntile::fp16_t, bit-compatible with __half) forms of every fused-pair
 * entry point above and of the tensor-level loops below: same arguments, contracts,
 * shapes and status word; the mask holds fp16 values (0, -inf = 0xFC00, or any finite
 * bias); P, dS and all outputs are rounded to fp16 where the bfloat16 forms round to
 * bf16.  The reference instantiates its codelets and cuDNN wrappers for both types
 * (src/starpu/flash_sdpa_fwd_cudnn.cc:292-293, src/starpu/flash_sdpa_bwd_cudnn.cc,
 * src/kernel/flash_sdpa_fwd_cudnn/cuda.cc:53-63). */
int nntile_b200_flash_sdpa_fwd_fp16(nntile_b200_stream_t stream, int64_t seq,
        int64_t head, int64_t batch, const void *K, const void *Q,
        const void *mask, float *scratch_lse, const void *V, void *scratch_A,
        float *lse, void *A);
int nntile_b200_flash_sdpa_bwd_fp16(nntile_b200_stream_t stream, int64_t seq,
        int64_t head, int64_t batch, const void *K, const void *Q, const void *V,
        const void *A, const void *dA, const void *mask, const float *lse,
        void *scratch_dK, void *scratch_dQ, void *scratch_dV, void *dK, void *dQ,
        void *dV);
int nntile_b200_flash_sdpa_fwd_gqa_fp16(nntile_b200_stream_t stream, int64_t seq,
        int64_t head, int64_t batch, int64_t group, int64_t kv_heads, const void *K,
        const void *Q, const void *mask, const void *V, float *lse, void *A,
        void *scratch, size_t scratch_bytes);
int nntile_b200_flash_sdpa_bwd_gqa_fp16(nntile_b200_stream_t stream, int64_t seq,
        int64_t head, int64_t batch, int64_t group, int64_t kv_heads, const void *K,
        const void *Q, const void *V, const void *A, const void *dA, const void *mask,
        const float *lse, void *dK, void *dQ, void *dV, void *scratch,
        size_t scratch_bytes);
int nntile_b200_tensor_flash_sdpa_fwd_fp16(nntile_b200_stream_t stream,
        const int64_t *shape, const int64_t *basetile, const void *const *K_tiles,
        const void *const *Q_tiles, const void *const *mask_tiles,
        float *const *lse_tiles, const void *const *V_tiles, void *const *A_tiles,
        void *scratch, size_t scratch_bytes);
int nntile_b200_tensor_flash_sdpa_bwd_fp16(nntile_b200_stream_t stream,
        const int64_t *shape, const int64_t *basetile, const void *const *K_tiles,
        const void *const *Q_tiles, const void *const *V_tiles,
        const void *const *A_tiles, const void *const *dA_tiles,
        const void *const *mask_tiles, const float *const *lse_tiles,
        void *const *dK_tiles, void *const *dQ_tiles, void *const *dV_tiles,
        void *scratch, size_t scratch_bytes);
int nntile_b200_tensor_flash_sdpa_fwd_gqa_fp16(nntile_b200_stream_t stream,
        const int64_t *shape, const int64_t *basetile, const void *const *K_tiles,
        const void *const *Q_tiles, const void *const *mask_tiles,
        float *const *lse_tiles, const void *const *V_tiles, void *const *A_tiles,
        void *scratch, size_t scratch_bytes);
int nntile_b200_tensor_flash_sdpa_bwd_gqa_fp16(nntile_b200_stream_t stream,
        const int64_t *shape, const int64_t *basetile, const void *const *K_tiles,
        const void *const *Q_tiles, const void *const *V_tiles,
        const void *const *A_tiles, const void *const *dA_tiles,
        const void *const *mask_tiles, const float *const *lse_tiles,
        void *const *dK_tiles, void *const *dQ_tiles, void *const *dV_tiles,
        void *scratch, size_t scratch_bytes);

/* Which implementation nntile_b200_flash_sdpa_{fwd,bwd}_bf16 pick for a shape:
 * 2 = tcgen05/TMEM/TMA kernel, 1 = generic CUDA kernel, 0 = rejected. */
int nntile_b200_flash_sdpa_fwd_path(int64_t seq, int64_t head, int64_t batch);
int nntile_b200_flash_sdpa_bwd_path(int64_t seq, int64_t head, int64_t batch);

/* ---------------------------------------------------------------------------
 * Layout changes around the SDPA layer, fused with their neighbours
 * ------------------------------------------------------------------------- */

/* dst[head, seq, batch, lead] = RoPE(src[lead, head, seq, batch]): the projection
 * output (lead = group*kv_heads for Q, kv_heads for K, fastest index) brought into
 * the SDPA layout and rotated in one pass.  sin, cos: bf16 [head/2, seq, batch] as
 * the reference's attention layer fills them; both NULL = layout change only (V).
 *   dst[2i, .., n]   = cos[i,..]*x[2i] - sin[i,..]*x[2i+1]
 *   dst[2i+1, .., n] = sin[i,..]*x[2i] + cos[i,..]*x[2i+1],  x = src[n, :, ..]
 * fp32 arithmetic without fused multiply-add, one rounding to bf16: bit-identical to
 * the two reference passes.  lead even, head a multiple of 8, pointers 16-byte aligned.
 * Replaces transpose_async(1.0, src, tmp, ndim) followed by rope_async(sin, cos, tmp,
 * dst) (wrappers/python/nntile/model/llama_attention.py:592-625; kernels
 * nntile::kernel::transpose::cuda<T>, src/kernel/transpose/cuda.cu:24-132, and
 * nntile::kernel::rope::cuda<T>, src/kernel/rope/cuda.cu:21-57).  Together with the
 * grouped-query entry points below the K/V replication (add_slice_inplace, :605-616)
 * disappears as well. */
int nntile_b200_transpose_rope_bf16(nntile_b200_stream_t stream, int64_t lead,
        int64_t head, int64_t seq, int64_t batch, const void *sin, const void *cos,
        const void *src, void *dst);

/* dst[head, seq, batch, lead] = src[lead, head, seq, batch] + bias[head, lead]:
 * GPT-2's prologue, transpose_async + add_fiber_inplace_async(1.0, bias, 1.0, dst, 0, 1)
 * (wrappers/python/nntile/model/gpt2_attention.py:258-273; kernel
 * src/kernel/add_fiber_inplace/cuda.cu) in one pass, one rounding. */
int nntile_b200_transpose_bias_bf16(nntile_b200_stream_t stream, int64_t lead,
        int64_t head, int64_t seq, int64_t batch, const void *bias, const void *src,
        void *dst);

/* dst[lead, head, seq, batch] = src[head, seq, batch, lead]: the attention output
 * brought back for the output projection (transpose_async(1.0, A, At, 3),
 * llama_attention.py:620-623, gpt2_attention.py:270-272). */
int nntile_b200_transpose_heads_back_bf16(nntile_b200_stream_t stream, int64_t lead,
        int64_t head, int64_t seq, int64_t batch, const void *src, void *dst);

/* ---------------------------------------------------------------------------
 * Decode: one new query token against a KV cache, split over the cache length
 * ------------------------------------------------------------------------- */

/* out[head, 1, batch, group, kv_heads] = softmax(q.K^T/sqrt(head)) V over the first
 * `length` cache positions, reading the un-replicated cache once for all `group`
 * query heads of a KV head.  q/out: bf16 [head, 1, batch, group, kv_heads];
 * Kcache/Vcache: bf16 [head, max_seq, batch, kv_heads] (the reference's cache
 * layout, include/nntile/graph/kv_cache.hh:38-39); lse_out: optional fp32
 * [batch, group, kv_heads] (may be NULL).  `workspace` must hold at least
 * nntile_b200_decode_sdpa_workspace_bytes(...) bytes, 16-byte aligned.
 * Replaces the chain the reference runs for a non-empty cache (cache copy + K/V
 * replication + gemm/maxsumexp/softmax_inplace/gemm with one query position,
 * wrappers/python/nntile/model/llama_attention.py:533-616, 672-676,
 * wrappers/python/nntile/layer/sdpa.py:238-306). */
int nntile_b200_decode_sdpa_bf16(nntile_b200_stream_t stream, int64_t head,
        int64_t max_seq, int64_t length, int64_t batch, int64_t group,
        int64_t kv_heads, const void *q, const void *Kcache, const void *Vcache,
        void *out, float *lse_out, void *workspace, size_t workspace_bytes);
size_t nntile_b200_decode_sdpa_workspace_bytes(int64_t head, int64_t length,
        int64_t batch, int64_t group, int64_t kv_heads);

/* Append `new_seq` positions to a KV cache in place:
 * cache[:, cache_len : cache_len + new_seq, :, :] = src, with src bf16
 * [head, new_seq, batch, kv_heads] and cache bf16 [head, max_seq, batch, kv_heads].
 * Replaces the copy_intersection_async call of KVCache.append
 * (wrappers/python/nntile/layer/cache_utils.py:146-176; kernel
 * src/kernel/subcopy); together with nntile_b200_decode_sdpa_bf16 reading only the
 * first `length` positions it also makes KVCache.k_partial / v_partial
 * (cache_utils.py:178-214: a copy of the filled part per decode step) unnecessary.
 * Rejected with NNTILE_B200_E_BADARG when cache_len + new_seq > max_seq. */
int nntile_b200_kv_cache_append_bf16(nntile_b200_stream_t stream, int64_t head,
        int64_t max_seq, int64_t batch, int64_t kv_heads, int64_t cache_len,
        int64_t new_seq, const void *src, void *cache);

/* The same operation for callers that cannot hand over a workspace because they
 * cannot allocate device memory where they run: the body of a StarPU codelet or
 * of any other task-runtime worker callback (cudaMalloc there would serialise the
 * device and go behind the runtime's memory accounting), or a C host that only
 * holds device pointers someone else gave it.  No counterpart in the reference.
 * The workspace is a fixed array inside the library image,
 * nntile_b200_decode_sdpa_noalloc_max_bytes() bytes (32 MiB) of device memory that
 * every GPU which loads the library keeps until the process exits; a problem whose
 * nntile_b200_decode_sdpa_workspace_bytes(...) exceeds it is rejected with
 * NNTILE_B200_E_SCRATCH.  The call allocates nothing and frees nothing.  The first
 * call on each device looks up the array's device address (cudaGetSymbolAddress,
 * with that device current) before it enqueues anything, so make that first call
 * per device outside any stream capture.  All calls on one device share the one
 * array and the array keeps whatever the last call left in it: two calls whose
 * kernels may overlap on the GPU (different streams) race and must be ordered by
 * the caller; calls on the same stream are safe.  Arguments, layouts and results
 * are those of nntile_b200_decode_sdpa_bf16. */
int nntile_b200_decode_sdpa_noalloc_bf16(nntile_b200_stream_t stream, int64_t head,
        int64_t max_seq, int64_t length, int64_t batch, int64_t group,
        int64_t kv_heads, const void *q, const void *Kcache, const void *Vcache,
        void *out, float *lse_out);
size_t nntile_b200_decode_sdpa_noalloc_max_bytes(void);

/* ---------------------------------------------------------------------------
 * Tensor level: the tile loops of the fused path
 * ------------------------------------------------------------------------- */

/* K, Q, V, A (and dA, dK, dQ, dV) are tiled tensors of `shape` =
 * [head, seq, batch, group, kv_heads] cut into tiles of `basetile`; every tile is
 * a separate Fortran-order device buffer and `*_tiles[i]` is tile i in Fortran
 * order of the tile grid.  mask is [seq, seq] tiled [basetile[1], basetile[1]]
 * (tile (k, q) at k + q*nseq_tiles), lse is [seq, batch, group, kv_heads] tiled
 * like A without the head axis.  For every output tile, one tile task per K/V
 * sequence tile is enqueued in order, fully masked pairs included, as in the
 * reference - unless the caller says otherwise: a NULL entry in `mask_tiles` marks
 * its (K/V tile, Q tile) pair as fully masked and no task is generated for it
 * (under a causal mask 44 % of the pairs of config 4), and several entries may point
 * to the same buffer, so a causal mask needs one zero tile and one diagonal tile
 * instead of a dense [seq, seq] tensor.  The caller runs the prologue (lse = -inf,
 * A = 0) for the forward and provides `scratch` of
 * nntile_b200_tensor_flash_sdpa_scratch_bytes(shape, basetile) bytes, 256-byte
 * aligned (status word, mask class tables, and for the backward delta, lse*log2e and
 * an fp32 dQ accumulator for the whole tensor).
 * Scheduling: the reference gives every pair to StarPU, which overlaps tasks of
 * different output tiles.  Here the caller's stream forks into a per-device pool of
 * helper streams (created on the first call on a device) and joins again before the
 * call returns, so all work is ordered after what precedes the call on `stream` and
 * before what follows it.  Tasks that merge into the same (lse, A) run in K/V-tile
 * order; tasks that add into the same dK/dV tile run in Q-tile order; dQ of a Q tile
 * is summed in fp32 over all its K/V tiles and rounded into dQ once (the reference
 * rounds per task).  Every distinct mask buffer is classified once per call.
 * Replace nntile::tensor::flash_sdpa_fwd_cudnn_async<bf16_t>,
 * src/tensor/flash_sdpa_fwd_cudnn.cc:211-279 (+ src/tile/flash_sdpa_fwd_cudnn.cc:161-196)
 * and nntile::tensor::flash_sdpa_bwd_cudnn_async<bf16_t>,
 * src/tensor/flash_sdpa_bwd_cudnn.cc:154-246 (+ src/tile/flash_sdpa_bwd_cudnn.cc:90-136). */
int nntile_b200_tensor_flash_sdpa_fwd_bf16(nntile_b200_stream_t stream,
        const int64_t *shape, const int64_t *basetile, const void *const *K_tiles,
        const void *const *Q_tiles, const void *const *mask_tiles,
        float *const *lse_tiles, const void *const *V_tiles, void *const *A_tiles,
        void *scratch, size_t scratch_bytes);
int nntile_b200_tensor_flash_sdpa_bwd_bf16(nntile_b200_stream_t stream,
        const int64_t *shape, const int64_t *basetile, const void *const *K_tiles,
        const void *const *Q_tiles, const void *const *V_tiles,
        const void *const *A_tiles, const void *const *dA_tiles,
        const void *const *mask_tiles, const float *const *lse_tiles,
        void *const *dK_tiles, void *const *dQ_tiles, void *const *dV_tiles,
        void *scratch, size_t scratch_bytes);
size_t nntile_b200_tensor_flash_sdpa_scratch_bytes(const int64_t *shape,
        const int64_t *basetile);

/* Grouped-query form of the tensor-level loops: Q, A, dA, dQ, lse tiled as above,
 * K, V, dK, dV are [head, seq, batch, kv_heads] tensors tiled
 * [head, basetile[1], basetile[2], basetile[4]] (tile (s, b, h) at
 * s + nseq*(b + nbatch*h)), not replicated over the group - what the reference's
 * attention layers hold before add_slice_inplace replicates them
 * (wrappers/python/nntile/model/llama_attention.py:605-616).  tcgen05 shapes only. */
int nntile_b200_tensor_flash_sdpa_fwd_gqa_bf16(nntile_b200_stream_t stream,
        const int64_t *shape, const int64_t *basetile, const void *const *K_tiles,
        const void *const *Q_tiles, const void *const *mask_tiles,
        float *const *lse_tiles, const void *const *V_tiles, void *const *A_tiles,
        void *scratch, size_t scratch_bytes);
int nntile_b200_tensor_flash_sdpa_bwd_gqa_bf16(nntile_b200_stream_t stream,
        const int64_t *shape, const int64_t *basetile, const void *const *K_tiles,
        const void *const *Q_tiles, const void *const *V_tiles,
        const void *const *A_tiles, const void *const *dA_tiles,
        const void *const *mask_tiles, const float *const *lse_tiles,
        void *const *dK_tiles, void *const *dQ_tiles, void *const *dV_tiles,
        void *scratch, size_t scratch_bytes);

#ifdef __cplusplus
}
#endif
#endif /* NNTILE_B200_H */
