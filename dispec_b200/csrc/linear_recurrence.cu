// Linear attention as a recurrence over a matrix state, in 32-bit floats on the FMA units:
//
//     S_t = diag(a_t) S_(t-1) + b_t v_t^T        (S: [dim, vdim] per head and request)
//     o_t = S_t^T q_t
//
// The state of a request lives in its state slot between steps, so a prompt can be cut into
// portions anywhere and decoded tokens continue from what the prompt left.  What a_t, b_t and
// q_t are is the mixer's business; two forms are built in, both computed here from the raw
// rows of the mixer's fused projection (float or bfloat16), in 32-bit:
//
//   FIXED_DECAY   a_t = decay[head] (one number per head); q_t and b_t are the projected query
//                 and key with pairs (i, i + rot/2) of their first `rot` dimensions turned by
//                 the angle position * inv_freq[i], and b_t scaled by `key_scale` afterwards
//   FORGET_GATE   a_t = f_t = lower + (1 - lower) * sigmoid(raw_f + bias), b_t = 1 - f_t,
//                 q_t = silu(raw_q)      (lower and bias per head and channel)
//
// One block per (request, head, tile of value columns).  A thread holds ROWS state rows of one
// column in registers; the SLICES threads that share a column sit in adjacent lanes and add
// their partial outputs by shuffles.  Tokens are staged through shared memory in rounds of
// `tokens_per_round`, transformed as they are staged.  A request whose first row carries a
// negative position (a padding row of a captured step) is skipped: its state slot belongs to
// someone else.
#include "common.cuh"

namespace {

enum { FIXED_DECAY = 0, FORGET_GATE = 1 };

struct RecurrenceArgs {
  const void* proj;  // [T, ld]: raw projection rows
  int proj_dtype;
  long ld;
  int q_off, k_off, v_off;  // first column of the query, key (or forget gate) and value parts
  int mode;
  int H, dim, vdim;
  const float* decay;     // [H]                  FIXED_DECAY
  const float* inv_freq;  // [rot / 2]            FIXED_DECAY (may be null when rot == 0)
  int rot;
  float key_scale;
  const float* gate_bias;  // [H * dim]           FORGET_GATE
  const float* lower;      // [H * dim]           FORGET_GATE
  float* state;            // [slots, H, dim, vdim]
  const int* state_slot;   // [S]
  const int* q_start;      // [S + 1]
  const int* positions;    // [T]
  float* out;              // [T, ldo]: o_t at columns head * vdim + j
  long ldo;
  int slices;            // threads per column (a power of two, at most 32)
  int cols_per_block;    // threads / slices
  int tokens_per_round;
};

template <int ROWS>
__global__ void __launch_bounds__(128)
linear_recurrence_kernel(const RecurrenceArgs p) {
  extern __shared__ float smem[];
  pdl_launch_dependents();
  pdl_wait();
  const int seq = blockIdx.z, head = blockIdx.y;
  const int t0 = p.q_start[seq], t1 = p.q_start[seq + 1];
  if (t1 <= t0 || p.positions[t0] < 0) return;
  const int tid = threadIdx.x;
  const int slice = tid % p.slices, col_local = tid / p.slices;
  const int col = blockIdx.x * p.cols_per_block + col_local;
  const bool col_ok = col < p.vdim;
  const int dpad = p.slices * ROWS;  // state rows covered by the threads of a column (>= dim)
  const int R = p.tokens_per_round, C = p.cols_per_block;
  float* qs = smem;               // [R][dpad]
  float* bs = qs + R * dpad;      // [R][dpad]
  float* as = bs + R * dpad;      // [R][dpad]  (FORGET_GATE only)
  float* vs = as + (p.mode == FORGET_GATE ? R * dpad : 0);  // [R][C]
  float* os = vs + R * C;         // [R][C]

  float* sp = p.state + (((size_t)p.state_slot[seq] * p.H + head) * p.dim) * p.vdim;
  float S[ROWS];
#pragma unroll
  for (int k = 0; k < ROWS; ++k) {
    const int i = slice + p.slices * k;
    S[k] = (col_ok && i < p.dim) ? sp[(size_t)i * p.vdim + col] : 0.f;
  }
  const float decay = p.mode == FIXED_DECAY ? p.decay[head] : 0.f;
  const int half = p.rot / 2;

  for (int base = t0; base < t1; base += R) {
    const int n = min(R, t1 - base);
    __syncthreads();
    // stage and transform the round's tokens
    for (int idx = tid; idx < n * dpad; idx += blockDim.x) {
      const int r = idx / dpad, i = idx % dpad;
      const size_t rowp = (size_t)(base + r) * p.ld;
      float qv = 0.f, bv = 0.f, av = 0.f;
      if (i < p.dim) {
        const size_t qo = rowp + p.q_off + (size_t)head * p.dim, ko = rowp + p.k_off + (size_t)head * p.dim;
        if (p.mode == FIXED_DECAY) {
          qv = ld_any(p.proj, p.proj_dtype, qo + i);
          bv = ld_any(p.proj, p.proj_dtype, ko + i);
          if (i < p.rot) {
            const int f = i < half ? i : i - half;
            const int other = i < half ? i + half : i - half;
            float sn, cs;
            sincosf((float)p.positions[base + r] * p.inv_freq[f], &sn, &cs);
            const float q2 = ld_any(p.proj, p.proj_dtype, qo + other);
            const float k2 = ld_any(p.proj, p.proj_dtype, ko + other);
            // first of the pair: u cos - v sin; second: v cos + u sin
            qv = i < half ? qv * cs - q2 * sn : qv * cs + q2 * sn;
            bv = i < half ? bv * cs - k2 * sn : bv * cs + k2 * sn;
          }
          bv *= p.key_scale;
        } else {
          const float rq = ld_any(p.proj, p.proj_dtype, qo + i);
          qv = rq / (1.f + expf(-rq));
          const float rf = ld_any(p.proj, p.proj_dtype, ko + i) + p.gate_bias[head * p.dim + i];
          const float lo = p.lower[head * p.dim + i];
          av = lo + (1.f - lo) * (1.f / (1.f + expf(-rf)));
          bv = 1.f - av;
        }
      }
      qs[idx] = qv;
      bs[idx] = bv;
      if (p.mode == FORGET_GATE) as[idx] = av;
    }
    for (int idx = tid; idx < n * C; idx += blockDim.x) {
      const int r = idx / C, c = blockIdx.x * C + idx % C;
      vs[idx] = c < p.vdim ? ld_any(p.proj, p.proj_dtype, (size_t)(base + r) * p.ld + p.v_off + (size_t)head * p.vdim + c) : 0.f;
    }
    __syncthreads();
    for (int r = 0; r < n; ++r) {
      const float v = vs[r * C + col_local];
      const float* qr = qs + r * dpad + slice;
      const float* br = bs + r * dpad + slice;
      float acc = 0.f;
      if (p.mode == FORGET_GATE) {
        const float* ar = as + r * dpad + slice;
#pragma unroll
        for (int k = 0; k < ROWS; ++k) {
          S[k] = fmaf(ar[p.slices * k], S[k], br[p.slices * k] * v);
          acc = fmaf(S[k], qr[p.slices * k], acc);
        }
      } else {
#pragma unroll
        for (int k = 0; k < ROWS; ++k) {
          S[k] = fmaf(decay, S[k], br[p.slices * k] * v);
          acc = fmaf(S[k], qr[p.slices * k], acc);
        }
      }
      for (int o = 1; o < p.slices; o <<= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
      if (slice == 0) os[r * C + col_local] = acc;
    }
    __syncthreads();
    for (int idx = tid; idx < n * C; idx += blockDim.x) {
      const int r = idx / C, c = blockIdx.x * C + idx % C;
      if (c < p.vdim) p.out[(size_t)(base + r) * p.ldo + (size_t)head * p.vdim + c] = os[idx];
    }
  }
#pragma unroll
  for (int k = 0; k < ROWS; ++k) {
    const int i = slice + p.slices * k;
    if (col_ok && i < p.dim) sp[(size_t)i * p.vdim + col] = S[k];
  }
}

template <int ROWS>
int launch(const RecurrenceArgs& a, int S, size_t smem, cudaStream_t stream) {
  static size_t configured = 48 * 1024;
  if (smem > configured) {
    DSP_CUDA(cudaFuncSetAttribute(linear_recurrence_kernel<ROWS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    configured = smem;
  }
  dim3 grid((a.vdim + a.cols_per_block - 1) / a.cols_per_block, a.H, S);
  DSP_CUDA(launch_pdl(linear_recurrence_kernel<ROWS>, grid, dim3(128), smem, stream, a));
  DSP_CHECK_LAUNCH("dsp_linear_recurrence");
  return 0;
}
}  // namespace

extern "C" int dsp_linear_recurrence(const void* proj, int proj_dtype, long ld, int q_off, int k_off,
                                     int v_off, int mode, int H, int dim, int vdim, const float* decay,
                                     const float* inv_freq, int rot, float key_scale,
                                     const float* gate_bias, const float* lower, float* state,
                                     const int* state_slot, const int* q_start, const int* positions,
                                     float* out, long ldo, int S, cudaStream_t stream) {
  if (S == 0) return 0;
  DSP_REQUIRE(proj && state && state_slot && q_start && positions && out, "dsp_linear_recurrence: missing operand");
  DSP_REQUIRE(H > 0 && H <= 65535 && S <= 65535, "dsp_linear_recurrence: H=%d, S=%d outside the grid", H, S);
  DSP_REQUIRE(dim > 0 && dim <= 1024 && vdim > 0, "dsp_linear_recurrence: dim=%d (at most 1024), vdim=%d", dim, vdim);
  if (mode == FIXED_DECAY) {
    DSP_REQUIRE(decay != nullptr, "dsp_linear_recurrence: no decay");
    DSP_REQUIRE(rot >= 0 && rot <= dim && rot % 2 == 0 && (rot == 0 || inv_freq), "dsp_linear_recurrence: rot=%d", rot);
  } else if (mode == FORGET_GATE) {
    DSP_REQUIRE(gate_bias && lower, "dsp_linear_recurrence: no gate bias or lower bound");
  } else {
    DSP_REQUIRE(false, "dsp_linear_recurrence: unknown mode %d", mode);
  }
  RecurrenceArgs a;
  a.proj = proj; a.proj_dtype = proj_dtype; a.ld = ld;
  a.q_off = q_off; a.k_off = k_off; a.v_off = v_off; a.mode = mode;
  a.H = H; a.dim = dim; a.vdim = vdim;
  a.decay = decay; a.inv_freq = inv_freq; a.rot = rot; a.key_scale = key_scale;
  a.gate_bias = gate_bias; a.lower = lower;
  a.state = state; a.state_slot = state_slot; a.q_start = q_start; a.positions = positions;
  a.out = out; a.ldo = ldo;
  // threads per column: four, or as many as keep a thread's rows at 32 (a power of two)
  int slices = 4;
  while ((dim + slices - 1) / slices > 32) slices *= 2;
  const int rows = (dim + slices - 1) / slices;
  a.slices = slices;
  a.cols_per_block = 128 / slices;
  const int R = rows <= 8 ? 8 : (rows <= 16 ? 16 : 32);
  const int dpad = slices * R;
  a.tokens_per_round = dpad <= 128 ? 16 : 8;
  const size_t smem = sizeof(float) * ((size_t)a.tokens_per_round * dpad * (mode == FORGET_GATE ? 3 : 2) +
                                       (size_t)a.tokens_per_round * a.cols_per_block * 2);
  if (R == 8) return launch<8>(a, S, smem, stream);
  if (R == 16) return launch<16>(a, S, smem, stream);
  return launch<32>(a, S, smem, stream);
}
