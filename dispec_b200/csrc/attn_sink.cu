// Kernels of the attention mixer whose keys and values have widths of their own, whose values
// may be blended with another layer's values of the same token, and whose softmax may carry a
// sink (one more key of score 0 and no value).
//
// dsp_qkv_rotate_store: one block per token.  From a row [q (H x Dk) | k (G x Dk) | v (G x Dv)] of
// the fused projection (float or bfloat16) it
//   * turns pairs (i, i + rot/2), i < rot/2, of every query and key head by the angle
//     position * inv_freq[i] (32-bit angles, sine and cosine) and leaves the other dimensions,
//   * blends v <- (1 - lambda) v + lambda v_other when `v_other` is given (lambda read from the
//     device), in 32-bit,
//   * writes the turned query to `q_out` [T, H * Dk] and the turned key and the blended value to
//     the pages (pools [num_pages, G, page_size, Dk] and [.., Dv]) in the pools' type.
// A row with a negative position (padding of a captured step) is skipped; a page id outside the
// pool is recorded in the device error word and nothing is stored.
//
// dsp_attn_sink_mma_*: tensor-core attention over the same pools, see below.
#include "common.cuh"

namespace {

__global__ void __launch_bounds__(256)
qkv_rotate_store_kernel(const void* __restrict__ qkv, int in_dtype, long ld, const int* __restrict__ positions,
                        const int* __restrict__ seq_of_token, const int* __restrict__ page_table, int pt_stride,
                        void* __restrict__ k_pool, void* __restrict__ v_pool, int pool_dtype,
                        const float* __restrict__ inv_freq, int rot, const void* __restrict__ v_other, int vo_dtype,
                        long ld_vo, const float* __restrict__ lambda, void* __restrict__ q_out, long ld_q, int H,
                        int G, int Dk, int Dv, int page_size, int num_pages, int write_kv, int* err) {
  extern __shared__ float cs[];  // [rot/2] cosines, then [rot/2] sines
  const int t = blockIdx.x;
  const int pos = positions[t];
  if (pos < 0) return;
  const int half = rot / 2;
  for (int i = threadIdx.x; i < half; i += blockDim.x) sincosf((float)pos * inv_freq[i], &cs[half + i], &cs[i]);
  __syncthreads();
  const size_t row = (size_t)t * ld;
  auto turned = [&](size_t head0, int i) {
    const float v = ld_any(qkv, in_dtype, head0 + i);
    if (i >= rot) return v;
    if (i < half) return v * cs[i] - ld_any(qkv, in_dtype, head0 + i + half) * cs[half + i];
    return v * cs[i - half] + ld_any(qkv, in_dtype, head0 + i - half) * cs[half + i - half];
  };
  for (int idx = threadIdx.x; idx < H * Dk; idx += blockDim.x)
    st_any(q_out, pool_dtype, (size_t)t * ld_q + idx, turned(row + (size_t)(idx / Dk) * Dk, idx % Dk));
  if (!write_kv) return;
  const int page = page_table[(size_t)seq_of_token[t] * pt_stride + pos / page_size];
  if (page < 0 || page >= num_pages) {
    if (threadIdx.x == 0) atomicOr(err, DSP_ERR_BAD_PAGE);
    return;
  }
  const size_t k0 = row + (size_t)H * Dk, v0 = k0 + (size_t)G * Dk;
  for (int idx = threadIdx.x; idx < G * Dk; idx += blockDim.x) {
    const int g = idx / Dk, i = idx % Dk;
    const size_t dst = (((size_t)page * G + g) * page_size + pos % page_size) * Dk + i;
    st_any(k_pool, pool_dtype, dst, turned(k0 + (size_t)g * Dk, i));
  }
  const float lam = (v_other && lambda) ? *lambda : 0.f;
  for (int idx = threadIdx.x; idx < G * Dv; idx += blockDim.x) {
    const int g = idx / Dv, i = idx % Dv;
    float v = ld_any(qkv, in_dtype, v0 + idx);
    if (v_other) v = (1.f - lam) * v + lam * ld_any(v_other, vo_dtype, (size_t)t * ld_vo + idx);
    const size_t dst = (((size_t)page * G + g) * page_size + pos % page_size) * Dv + i;
    st_any(v_pool, pool_dtype, dst, v);
  }
}
}  // namespace

extern "C" int dsp_qkv_rotate_store(const void* qkv, int in_dtype, long ld, const int* positions,
                                    const int* seq_of_token, const int* page_table, int pt_stride, void* k_pool,
                                    void* v_pool, int pool_dtype, const float* inv_freq, int rot,
                                    const void* v_other, int vo_dtype, long ld_vo, const float* lambda, void* q_out,
                                    long ld_q, int T, int H, int G, int Dk, int Dv, int page_size, int num_pages,
                                    int write_kv, cudaStream_t stream) {
  if (T == 0) return 0;
  DSP_REQUIRE(qkv && positions && q_out && H > 0 && G > 0 && Dk > 0 && Dv > 0, "dsp_qkv_rotate_store: missing operand");
  DSP_REQUIRE(rot >= 0 && rot % 2 == 0 && rot <= Dk && (rot == 0 || inv_freq), "dsp_qkv_rotate_store: rot=%d for keys of %d", rot, Dk);
  DSP_REQUIRE(!write_kv || (k_pool && v_pool && page_table && seq_of_token && page_size > 0),
              "dsp_qkv_rotate_store: no pools to write to");
  DSP_REQUIRE(!v_other || lambda, "dsp_qkv_rotate_store: values to blend with but no weight");
  int* err = dsp_device_error_ptr();
  DSP_REQUIRE(err != nullptr, "dsp_qkv_rotate_store: no device error word");
  DSP_CUDA(launch_plain(qkv_rotate_store_kernel, dim3(T), dim3(256), (size_t)rot * sizeof(float), stream, qkv, in_dtype,
                        ld, positions, seq_of_token, page_table, pt_stride, k_pool, v_pool, pool_dtype, inv_freq, rot,
                        v_other, vo_dtype, ld_vo, lambda, q_out, ld_q, H, G, Dk, Dv, page_size, num_pages, write_kv,
                        err));
  DSP_CHECK_LAUNCH("dsp_qkv_rotate_store");
  return 0;
}
