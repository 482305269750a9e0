// Attention over a cached latent, all arithmetic in 32-bit.
//
// Every token leaves two rows in the paged cache: a latent c of R values (already normalised)
// and one rotated key part of r values that all heads share.  A head's unrotated key and its
// value are linear maps of c, so neither is ever materialised: the caller folds the key map
// into the query (qa = Wk^T q, R values per head) and applies the value map to the result, and
// this kernel computes, per query token at position p and head h,
//
//     s_j = scale * (qa_h . c_j + rot(qr_h, p) . kr_j)        for every cached j <= p
//     out_h = sum_j softmax(s)_j c_j                           (R values)
//
// which is attention with ONE key/value head of key width R + r and value width R.
//
// latent_store_kernel: RMS norm (32-bit) of the first R columns of the down projection with a
// gain, rotation of the last r columns, both written to the token's place in the pages.
// The rotation turns the pairs (2i, 2i+1) of the first `rot` of the r dimensions by the angle
// position * inv_freq[i] (interleaved layout); the rest pass unchanged.
//
// pools: latent [num_pages, 1, page_size, R], rotated key [num_pages, 1, page_size, r];
// page = page_table[seq * pt_stride + position / page_size].
#include "common.cuh"

namespace {
constexpr int THREADS = 128;  // = keys per tile
constexpr int GCHUNK = 8;     // heads per block

__global__ void __launch_bounds__(THREADS)
latent_store_kernel(const void* __restrict__ down, int d_dtype, long ldd, int c_off, int r_off,
                    const float* __restrict__ gain, float eps, const float* __restrict__ inv_freq,
                    int rot, const int* __restrict__ positions, const int* __restrict__ seq_of_token,
                    const int* __restrict__ page_table, int pt_stride, void* __restrict__ c_pool,
                    void* __restrict__ r_pool, int pool_dtype, int R, int r, int page_size,
                    int num_pages, int* err) {
  __shared__ float scratch[32];
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const int pos = positions[t];
  if (pos < 0) return;
  const int page = page_table[(size_t)seq_of_token[t] * pt_stride + pos / page_size];
  if (page < 0 || page >= num_pages) {
    if (threadIdx.x == 0) atomicOr(err, DSP_ERR_BAD_PAGE);
    return;
  }
  const size_t place = (size_t)page * page_size + pos % page_size;
  const size_t row = (size_t)t * ldd;
  float ss = 0.f;
  for (int i = threadIdx.x; i < R; i += THREADS) {
    const float v = ld_any(down, d_dtype, row + c_off + i);
    ss = fmaf(v, v, ss);
  }
  const float inv = 1.f / sqrtf(block_sum(ss, scratch) / (float)R + eps);
  for (int i = threadIdx.x; i < R; i += THREADS)
    st_any(c_pool, pool_dtype, place * R + i, ld_any(down, d_dtype, row + c_off + i) * inv * gain[i]);
  for (int i = threadIdx.x; i < r; i += THREADS) {
    float v = ld_any(down, d_dtype, row + r_off + i);
    if (i < rot) {
      float sn, cs;
      sincosf((float)pos * inv_freq[i >> 1], &sn, &cs);
      const float other = ld_any(down, d_dtype, row + r_off + (i ^ 1));
      v = (i & 1) ? v * cs + other * sn : v * cs - other * sn;
    }
    st_any(r_pool, pool_dtype, place * r + i, v);
  }
}

// One block per (query token, chunk of GCHUNK heads); a thread scores one key of the tile for
// every head of the chunk, then owns output dimensions tid, tid + 128, ...
template <typename T, int DPT>
__global__ void __launch_bounds__(THREADS)
attn_latent_kernel(const float* __restrict__ qa, long ldqa, const void* __restrict__ q, int q_dtype,
                   long ldq, int q_head_stride, int qr_off, const float* __restrict__ inv_freq, int rot,
                   const T* __restrict__ c_pool, const T* __restrict__ r_pool,
                   const int* __restrict__ page_table, int pt_stride, const int* __restrict__ positions,
                   const int* __restrict__ seq_of_token, void* __restrict__ out, int out_dtype, long ldo,
                   int H, int R, int r, int page_size, int num_pages, float scale, int* err) {
  extern __shared__ float smem[];
  const int W = R + r;
  float* qs = smem;                        // [GCHUNK][W]
  float* ps = qs + GCHUNK * W;             // [GCHUNK][THREADS]
  long* place = (long*)(ps + GCHUNK * THREADS);  // [THREADS] row of each key in the pools
  __shared__ float red[GCHUNK][THREADS / 32];
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x, h0 = blockIdx.y * GCHUNK;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int pos = positions[t];
  if (pos < 0) return;
  const int* table = page_table + (size_t)seq_of_token[t] * pt_stride;
  const int gn = min(GCHUNK, H - h0);

  for (int i = tid; i < gn * W; i += THREADS) {
    const int g = i / W, d = i % W;
    float v;
    if (d < R) {
      v = qa[(size_t)t * ldqa + (size_t)(h0 + g) * R + d];
    } else {
      const int j = d - R;
      const size_t at = (size_t)t * ldq + (size_t)(h0 + g) * q_head_stride + qr_off;
      v = ld_any(q, q_dtype, at + j);
      if (j < rot) {
        float sn, cs;
        sincosf((float)pos * inv_freq[j >> 1], &sn, &cs);
        const float other = ld_any(q, q_dtype, at + (j ^ 1));
        v = (j & 1) ? v * cs + other * sn : v * cs - other * sn;
      }
    }
    qs[i] = v * scale;
  }
  float m[GCHUNK], l[GCHUNK], acc[GCHUNK][DPT];
#pragma unroll
  for (int g = 0; g < GCHUNK; ++g) {
    m[g] = -INFINITY;
    l[g] = 0.f;
#pragma unroll
    for (int j = 0; j < DPT; ++j) acc[g][j] = 0.f;
  }
  __syncthreads();

  for (int kt = 0; kt <= pos; kt += THREADS) {
    const int key = kt + tid;
    float s[GCHUNK];
#pragma unroll
    for (int g = 0; g < GCHUNK; ++g) s[g] = -INFINITY;
    long at = -1;
    if (key <= pos) {
      const int page = table[key / page_size];
      if (page < 0 || page >= num_pages) {
        atomicOr(err, DSP_ERR_BAD_PAGE);
      } else {
        at = (long)page * page_size + key % page_size;
        const T* cr = c_pool + at * R;
        const T* rr = r_pool + at * r;
#pragma unroll
        for (int g = 0; g < GCHUNK; ++g) s[g] = 0.f;
        for (int d = 0; d < R; ++d) {
          const float kv = to_f32(cr[d]);
#pragma unroll
          for (int g = 0; g < GCHUNK; ++g)
            if (g < gn) s[g] = fmaf(qs[g * W + d], kv, s[g]);
        }
        for (int d = 0; d < r; ++d) {
          const float kv = to_f32(rr[d]);
#pragma unroll
          for (int g = 0; g < GCHUNK; ++g)
            if (g < gn) s[g] = fmaf(qs[g * W + R + d], kv, s[g]);
        }
      }
    }
    place[tid] = at;
#pragma unroll
    for (int g = 0; g < GCHUNK; ++g) {
      const float wm = warp_max(s[g]);
      if (lane == 0) red[g][warp] = wm;
    }
    __syncthreads();
    float alpha[GCHUNK], p[GCHUNK];
#pragma unroll
    for (int g = 0; g < GCHUNK; ++g) {
      float tm = red[g][0];
#pragma unroll
      for (int w = 1; w < THREADS / 32; ++w) tm = fmaxf(tm, red[g][w]);
      const float m_new = fmaxf(m[g], tm);
      alpha[g] = (m_new == -INFINITY) ? 1.f : expf(m[g] - m_new);
      p[g] = (at >= 0 && g < gn) ? expf(s[g] - m_new) : 0.f;
      m[g] = m_new;
      ps[g * THREADS + tid] = p[g];
    }
    __syncthreads();
#pragma unroll
    for (int g = 0; g < GCHUNK; ++g) {
      const float ws = warp_sum(p[g]);
      if (lane == 0) red[g][warp] = ws;
    }
    __syncthreads();
#pragma unroll
    for (int g = 0; g < GCHUNK; ++g) {
      float ts = red[g][0];
#pragma unroll
      for (int w = 1; w < THREADS / 32; ++w) ts += red[g][w];
      l[g] = l[g] * alpha[g] + ts;
#pragma unroll
      for (int j = 0; j < DPT; ++j) acc[g][j] *= alpha[g];
    }
    const int nkeys = min(THREADS, pos - kt + 1);
    for (int j = 0; j < nkeys; ++j) {
      const long vo = place[j];
      if (vo < 0) continue;
      const T* vr = c_pool + vo * R;
#pragma unroll
      for (int dd = 0; dd < DPT; ++dd) {
        const int d = tid + dd * THREADS;
        if (d < R) {
          const float vv = to_f32(vr[d]);
#pragma unroll
          for (int g = 0; g < GCHUNK; ++g)
            if (g < gn) acc[g][dd] = fmaf(ps[g * THREADS + j], vv, acc[g][dd]);
        }
      }
    }
    __syncthreads();
  }
#pragma unroll
  for (int g = 0; g < GCHUNK; ++g) {
    if (g >= gn) continue;
    const float inv = l[g] > 0.f ? 1.f / l[g] : 0.f;
#pragma unroll
    for (int dd = 0; dd < DPT; ++dd) {
      const int d = tid + dd * THREADS;
      if (d < R) st_any(out, out_dtype, (size_t)t * ldo + (size_t)(h0 + g) * R + d, acc[g][dd] * inv);
    }
  }
}

template <typename T, int DPT>
int launch_attn(const float* qa, long ldqa, const void* q, int q_dtype, long ldq, int q_head_stride,
                int qr_off, const float* inv_freq, int rot, const void* c_pool, const void* r_pool,
                const int* page_table, int pt_stride, const int* positions, const int* seq_of_token,
                void* out, int out_dtype, long ldo, int T_, int H, int R, int r, int page_size,
                int num_pages, float scale, int* err, cudaStream_t stream) {
  const size_t smem = (size_t)(GCHUNK * (R + r) + GCHUNK * THREADS) * sizeof(float) + THREADS * sizeof(long);
  static size_t configured = 48 * 1024;
  if (smem > configured) {
    DSP_CUDA(cudaFuncSetAttribute(attn_latent_kernel<T, DPT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    configured = smem;
  }
  dim3 grid(T_, (H + GCHUNK - 1) / GCHUNK);
  DSP_CUDA(launch_pdl(attn_latent_kernel<T, DPT>, grid, dim3(THREADS), smem, stream, qa, ldqa, q, q_dtype,
                      ldq, q_head_stride, qr_off, inv_freq, rot, (const T*)c_pool, (const T*)r_pool,
                      page_table, pt_stride, positions, seq_of_token, out, out_dtype, ldo, H, R, r,
                      page_size, num_pages, scale, err));
  DSP_CHECK_LAUNCH("dsp_attn_latent");
  return 0;
}
}  // namespace

extern "C" int dsp_latent_store(const void* down, int d_dtype, long ldd, int c_off, int r_off,
                                const float* gain, float eps, const float* inv_freq, int rot,
                                const int* positions, const int* seq_of_token, const int* page_table,
                                int pt_stride, void* c_pool, void* r_pool, int pool_dtype, int T_, int R,
                                int r, int page_size, int num_pages, cudaStream_t stream) {
  if (T_ == 0) return 0;
  int* err = dsp_device_error_ptr();
  DSP_REQUIRE(err != nullptr, "dsp_latent_store: no device error word");
  DSP_REQUIRE(down && gain && c_pool && r_pool && R > 0 && r >= 0, "dsp_latent_store: missing operand");
  DSP_REQUIRE(rot >= 0 && rot <= r && rot % 2 == 0 && (rot == 0 || inv_freq), "dsp_latent_store: rot=%d of %d", rot, r);
  DSP_CUDA(launch_pdl(latent_store_kernel, dim3(T_), dim3(THREADS), 0, stream, down, d_dtype, ldd, c_off,
                      r_off, gain, eps, inv_freq, rot, positions, seq_of_token, page_table, pt_stride,
                      c_pool, r_pool, pool_dtype, R, r, page_size, num_pages, err));
  DSP_CHECK_LAUNCH("dsp_latent_store");
  return 0;
}

extern "C" int dsp_attn_latent(const float* qa, long ldqa, const void* q, int q_dtype, long ldq,
                               int q_head_stride, int qr_off, const float* inv_freq, int rot,
                               const void* c_pool, const void* r_pool, int pool_dtype,
                               const int* page_table, int pt_stride, const int* positions,
                               const int* seq_of_token, void* out, int out_dtype, long ldo, int T_, int H,
                               int R, int r, int page_size, int num_pages, float scale,
                               cudaStream_t stream) {
  if (T_ == 0) return 0;
  int* err = dsp_device_error_ptr();
  DSP_REQUIRE(err != nullptr, "dsp_attn_latent: no device error word");
  DSP_REQUIRE(qa && q && c_pool && r_pool && out, "dsp_attn_latent: missing operand");
  DSP_REQUIRE(H > 0 && (H + GCHUNK - 1) / GCHUNK <= 65535, "dsp_attn_latent: H=%d", H);
  DSP_REQUIRE(R > 0 && R <= THREADS * 8, "dsp_attn_latent: latent size %d outside (0, %d]", R, THREADS * 8);
  DSP_REQUIRE(rot >= 0 && rot <= r && rot % 2 == 0 && (rot == 0 || inv_freq), "dsp_attn_latent: rot=%d of %d", rot, r);
#define DSP_LATENT_ARGS qa, ldqa, q, q_dtype, ldq, q_head_stride, qr_off, inv_freq, rot, c_pool, r_pool, page_table, \
                        pt_stride, positions, seq_of_token, out, out_dtype, ldo, T_, H, R, r, page_size, num_pages,  \
                        scale, err, stream
  const int dpt = (R + THREADS - 1) / THREADS;
  if (pool_dtype == DSP_F32) {
    if (dpt <= 1) return launch_attn<float, 1>(DSP_LATENT_ARGS);
    if (dpt <= 2) return launch_attn<float, 2>(DSP_LATENT_ARGS);
    if (dpt <= 4) return launch_attn<float, 4>(DSP_LATENT_ARGS);
    return launch_attn<float, 8>(DSP_LATENT_ARGS);
  }
  if (pool_dtype == DSP_BF16) {
    if (dpt <= 1) return launch_attn<bf16, 1>(DSP_LATENT_ARGS);
    if (dpt <= 2) return launch_attn<bf16, 2>(DSP_LATENT_ARGS);
    if (dpt <= 4) return launch_attn<bf16, 4>(DSP_LATENT_ARGS);
    return launch_attn<bf16, 8>(DSP_LATENT_ARGS);
  }
#undef DSP_LATENT_ARGS
  DSP_REQUIRE(false, "dsp_attn_latent: unknown pool dtype %d", pool_dtype);
}
