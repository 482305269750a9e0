// Row-wise kernels around a residual stream that is kept in 32-bit floats: the RMS norm of a
// scaled sum (the arrangement with the norm after the sum), the per-head RMS norm with an
// optional gain and gate that closes a linear-attention mixer, and the xIELU activation.
// All arithmetic is 32-bit; each operand has its own storage type (float or bfloat16).
#include "common.cuh"

namespace {

// y = w * s / sqrt(mean(s^2) + eps),   s = alpha * x + delta   (delta optional)
// `rows` (optional) gathers input rows.  y goes to y32 (float) and/or y16 (any type); y32 may
// be x itself.  One block per row, the row held in shared memory between the two passes.
__global__ void __launch_bounds__(256)
sum_norm_kernel(const void* __restrict__ x, int x_dtype, long ldx, const void* __restrict__ delta,
                int d_dtype, long ldd, const float* __restrict__ w, float alpha, float eps,
                const int* __restrict__ rows, float* y32, long ld32, void* __restrict__ y16,
                int y_dtype, long ld16, int width) {
  extern __shared__ float row[];
  __shared__ float scratch[32];
  const int r = blockIdx.x;
  const size_t in_row = rows ? (size_t)rows[r] : (size_t)r;
  float ss = 0.f;
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    float s = alpha * ld_any(x, x_dtype, in_row * ldx + i);
    if (delta) s += ld_any(delta, d_dtype, in_row * ldd + i);
    row[i] = s;
    ss = fmaf(s, s, ss);
  }
  const float total = block_sum(ss, scratch);
  const float inv = 1.f / sqrtf(total / (float)width + eps);
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    const float y = row[i] * inv * w[i];
    if (y32) y32[(size_t)r * ld32 + i] = y;
    if (y16) st_any(y16, y_dtype, (size_t)r * ld16 + i, y);
  }
}

// Per (token, head): y = o / sqrt(mean(o^2) + eps) * gain[j] * silu(gate[t, head, j])
// (gain and gate optional).  o is float [T, H * dv]; one warp per (token, head).
__global__ void __launch_bounds__(128)
head_norm_gate_kernel(const float* __restrict__ o, long ldo, const float* __restrict__ gain,
                      const void* __restrict__ gate, int g_dtype, long ldg, void* __restrict__ y,
                      int y_dtype, long ldy, int T, int H, int dv, float eps) {
  const int lane = threadIdx.x & 31;
  const long pair = (long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (pair >= (long)T * H) return;
  const int t = (int)(pair / H), h = (int)(pair % H);
  const float* row = o + (size_t)t * ldo + (size_t)h * dv;
  float ss = 0.f;
  for (int j = lane; j < dv; j += 32) ss = fmaf(row[j], row[j], ss);
  ss = warp_sum(ss);
  const float inv = 1.f / sqrtf(ss / (float)dv + eps);
  for (int j = lane; j < dv; j += 32) {
    float v = row[j] * inv;
    if (gain) v *= gain[j];
    if (gate) {
      const float g = ld_any(gate, g_dtype, (size_t)t * ldg + (size_t)h * dv + j);
      v *= g / (1.f + expf(-g));
    }
    st_any(y, y_dtype, (size_t)t * ldy + (size_t)h * dv + j, v);
  }
}

__device__ __forceinline__ float softplus_f(float v) { return v > 20.f ? v : log1pf(expf(v)); }

// xIELU with the two raw parameters (p, q) read from the device:
//   z > 0:  softplus(p) z^2 + z / 2
//   z <= 0: (1/2 + softplus(q)) (exp(z) - 1 - z) + z / 2
__global__ void __launch_bounds__(256)
xielu_kernel(const void* __restrict__ z, int z_dtype, long ldz, const float* __restrict__ pq,
             void* __restrict__ y, int y_dtype, long ldy, long rows, int cols) {
  const float ap = softplus_f(pq[0]), an = 0.5f + softplus_f(pq[1]);
  auto act = [&](float v) { return v > 0.f ? fmaf(ap * v, v, 0.5f * v) : fmaf(an, expm1f(v) - v, 0.5f * v); };
  // four elements a thread where rows are whole groups of four on 16-byte (8-byte) pieces
  const bool vec = z_dtype == DSP_F32 && y_dtype == DSP_BF16 && cols % 4 == 0 && ldz % 4 == 0 && ldy % 4 == 0 &&
                   ((uintptr_t)z % 16) == 0 && ((uintptr_t)y % 8) == 0;
  if (vec) {
    const int c4 = cols / 4;
    const long n = rows * c4;
    for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long)gridDim.x * blockDim.x) {
      const long r = i / c4;
      const int c = (int)(i % c4) * 4;
      const float4 v = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(z) + (size_t)r * ldz + c);
      __nv_bfloat162 lo = __floats2bfloat162_rn(act(v.x), act(v.y)), hi = __floats2bfloat162_rn(act(v.z), act(v.w));
      uint2 out;
      out.x = *reinterpret_cast<uint32_t*>(&lo);
      out.y = *reinterpret_cast<uint32_t*>(&hi);
      *reinterpret_cast<uint2*>(reinterpret_cast<bf16*>(y) + (size_t)r * ldy + c) = out;
    }
    return;
  }
  const long n = rows * cols;
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long)gridDim.x * blockDim.x) {
    const long r = i / cols;
    const int c = (int)(i % cols);
    st_any(y, y_dtype, (size_t)r * ldy + c, act(ld_any(z, z_dtype, (size_t)r * ldz + c)));
  }
}
}  // namespace

extern "C" int dsp_sum_norm(const void* x, int x_dtype, long ldx, const void* delta, int d_dtype,
                            long ldd, const float* w, float alpha, float eps, const int* rows,
                            float* y32, long ld32, void* y16, int y_dtype, long ld16, int n_rows,
                            int width, cudaStream_t stream) {
  if (n_rows == 0) return 0;
  DSP_REQUIRE(x && w && width > 0 && (y32 || y16), "dsp_sum_norm: missing operand");
  const size_t smem = (size_t)width * sizeof(float);
  DSP_REQUIRE(smem <= 200 * 1024, "dsp_sum_norm: a row of %d values does not fit shared memory", width);
  static size_t configured = 48 * 1024;
  if (smem > configured) {
    DSP_CUDA(cudaFuncSetAttribute(sum_norm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    configured = smem;
  }
  DSP_CUDA(launch_plain(sum_norm_kernel, dim3(n_rows), dim3(256), smem, stream, x, x_dtype, ldx, delta,
                      d_dtype, ldd, w, alpha, eps, rows, y32, ld32, y16, y_dtype, ld16, width));
  DSP_CHECK_LAUNCH("dsp_sum_norm");
  return 0;
}

extern "C" int dsp_head_norm_gate(const float* o, long ldo, const float* gain, const void* gate,
                                  int g_dtype, long ldg, void* y, int y_dtype, long ldy, int T, int H,
                                  int dv, float eps, cudaStream_t stream) {
  if (T == 0) return 0;
  DSP_REQUIRE(o && y && H > 0 && dv > 0, "dsp_head_norm_gate: missing operand");
  const long pairs = (long)T * H;
  DSP_CUDA(launch_plain(head_norm_gate_kernel, dim3((unsigned)((pairs + 3) / 4)), dim3(128), 0, stream, o,
                      ldo, gain, gate, g_dtype, ldg, y, y_dtype, ldy, T, H, dv, eps));
  DSP_CHECK_LAUNCH("dsp_head_norm_gate");
  return 0;
}

extern "C" int dsp_xielu(const void* z, int z_dtype, long ldz, const float* pq, void* y, int y_dtype,
                         long ldy, long rows, int cols, cudaStream_t stream) {
  if (rows == 0 || cols == 0) return 0;
  DSP_REQUIRE(z && pq && y, "dsp_xielu: missing operand");
  const long n = rows * cols;
  const int sms = dsp_num_sms();
  const long want = (n + 255) / 256, cap = (long)(sms > 0 ? sms : 148) * 16;
  DSP_CUDA(launch_plain(xielu_kernel, dim3((unsigned)(want < cap ? want : cap)), dim3(256), 0, stream, z,
                      z_dtype, ldz, pq, y, y_dtype, ldy, rows, cols));
  DSP_CHECK_LAUNCH("dsp_xielu");
  return 0;
}
