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
//                 the angle position * inv_freq[i], and b_t scaled by `key_scale` afterwards;
//                 with `act` = 1 the raw query, key and value pass through silu first
//   FORGET_GATE   a_t = f_t = lower + (1 - lower) * sigmoid(raw_f + bias), b_t = 1 - f_t,
//                 q_t = silu(raw_q)      (lower and bias per head and channel)
//
// One block per (request, head, tile of value columns).  A thread holds ROWS state rows of one
// column in registers; the SLICES threads that share a column sit in adjacent lanes and add
// their partial outputs by shuffles.  Tokens are staged through shared memory in rounds of
// `tokens_per_round`.  The recurrence is sequential in the tokens of a request, so what can be
// done ahead of it is: for portions of prompts a first, fully parallel kernel writes q_t, b_t
// (and a_t) of every token as floats, and the recurrence kernel only streams them in with
// cp.async, the next round arriving while the current one is computed; single tokens are
// transformed as they are staged, in one kernel.  A request whose first row carries a negative
// position (a padding row of a captured step) is skipped: its state slot belongs to someone else.
#include "common.cuh"

namespace {

enum { FIXED_DECAY = 0, FORGET_GATE = 1 };
constexpr int THREADS = 256;

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
  int act;  // 1: silu on the raw query, key and value (FIXED_DECAY)
  const float* gate_bias;  // [H * dim]           FORGET_GATE
  const float* lower;      // [H * dim]           FORGET_GATE
  float* state;            // [slots, H, dim, vdim]
  const int* state_slot;   // [S]
  const int* q_start;      // [S + 1]
  const int* positions;    // [T]
  float* out;              // [T, ldo]: o_t at columns head * vdim + j
  long ldo;
  float* ready;          // [T, planes, H * dim] floats written by the first kernel (null: transform while staging)
  int slices;            // threads per column (a power of two, at most 32)
  int cols_per_block;    // threads / slices
  int tokens_per_round;
};

// q_t, b_t and a_t of element (token, head, i) from the raw projection row, in 32-bit.
__device__ __forceinline__ void transform(const RecurrenceArgs& p, int token, int head, int i, float& qv,
                                          float& bv, float& av) {
  const size_t rowp = (size_t)token * p.ld;
  const size_t qo = rowp + p.q_off + (size_t)head * p.dim, ko = rowp + p.k_off + (size_t)head * p.dim;
  av = 0.f;
  if (p.mode == FIXED_DECAY) {
    qv = ld_any(p.proj, p.proj_dtype, qo + i);
    bv = ld_any(p.proj, p.proj_dtype, ko + i);
    if (p.act == 1) {
      qv = qv / (1.f + expf(-qv));
      bv = bv / (1.f + expf(-bv));
    }
    if (i < p.rot) {
      const int half = p.rot / 2;
      const int f = i < half ? i : i - half;
      const int other = i < half ? i + half : i - half;
      float sn, cs;
      sincosf((float)p.positions[token] * p.inv_freq[f], &sn, &cs);
      float q2 = ld_any(p.proj, p.proj_dtype, qo + other);
      float k2 = ld_any(p.proj, p.proj_dtype, ko + other);
      if (p.act == 1) {
        q2 = q2 / (1.f + expf(-q2));
        k2 = k2 / (1.f + expf(-k2));
      }
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

// ready[t][0] = q, [1] = b, [2] = a (FORGET_GATE only), each [H * dim]
__global__ void __launch_bounds__(256) recurrence_prepare_kernel(const RecurrenceArgs p, int T) {
  const int hd = p.H * p.dim, planes = p.mode == FORGET_GATE ? 3 : 2;
  const long n = (long)T * hd;
  for (long idx = (long)blockIdx.x * blockDim.x + threadIdx.x; idx < n; idx += (long)gridDim.x * blockDim.x) {
    const int t = (int)(idx / hd), c = (int)(idx % hd);
    if (p.positions[t] < 0) continue;
    float qv, bv, av;
    transform(p, t, c / p.dim, c % p.dim, qv, bv, av);
    float* dst = p.ready + (size_t)t * planes * hd + c;
    dst[0] = qv;
    dst[hd] = bv;
    if (planes == 3) dst[2 * hd] = av;
  }
}

__device__ __forceinline__ void cp_async4(float* smem, const float* gmem) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;\n" ::"r"((uint32_t)__cvta_generic_to_shared(smem)), "l"(gmem));
}

__device__ __forceinline__ void cp_async16(float* smem, const float* gmem) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"((uint32_t)__cvta_generic_to_shared(smem)), "l"(gmem));
}

// ROWS: state rows a thread holds; TPR: tokens per staging round
template <int ROWS, int TPR>
__global__ void __launch_bounds__(THREADS)
linear_recurrence_kernel(const RecurrenceArgs p) {
  extern __shared__ float smem[];
  const int seq = blockIdx.z, head = blockIdx.y;
  const int t0 = p.q_start[seq], t1 = p.q_start[seq + 1];
  if (t1 <= t0 || p.positions[t0] < 0) return;
  const int tid = threadIdx.x;
  const int slice = tid % p.slices, col_local = tid / p.slices;
  const int col = blockIdx.x * p.cols_per_block + col_local;
  const bool col_ok = col < p.vdim;
  const int dpad = p.slices * ROWS;  // state rows covered by the threads of a column (>= dim)
  constexpr int R = TPR;
  const int C = p.cols_per_block;
  const bool gate = p.mode == FORGET_GATE;
  const int planes = gate ? 3 : 2;
  // one staging buffer: [planes][R][dpad] then v [R][C]; two of them when rounds arrive by cp.async
  const int buf_floats = planes * R * dpad + R * C;
  float* os = smem + (p.ready ? 2 : 1) * buf_floats;  // [R][C]

  float* sp = p.state + (((size_t)p.state_slot[seq] * p.H + head) * p.dim) * p.vdim;
  float S[ROWS];
#pragma unroll
  for (int k = 0; k < ROWS; ++k) {
    const int i = slice + p.slices * k;
    S[k] = (col_ok && i < p.dim) ? sp[(size_t)i * p.vdim + col] : 0.f;
  }
  const float decay = gate ? 0.f : p.decay[head];
  const int hd = p.H * p.dim;

  // rows beyond dim stay zero in every buffer: they are written here once and never again
  if (dpad > p.dim)
    for (int idx = tid; idx < (p.ready ? 2 : 1) * buf_floats; idx += THREADS) smem[idx] = 0.f;
  __syncthreads();

  // rows of 16-byte pieces where every address allows it, single floats otherwise
  const bool wide = p.dim % 4 == 0 && (((uintptr_t)p.ready) & 15) == 0;
  auto stage_async = [&](int base, float* buf) {
    const int n = min(R, t1 - base);
    for (int pl = 0; pl < planes; ++pl)
      for (int r = tid >> 5; r < n; r += THREADS / 32) {
        float* dst = buf + (pl * R + r) * dpad;
        const float* src = p.ready + ((size_t)(base + r) * planes + pl) * hd + head * p.dim;
        if (wide)
          for (int i = (tid & 31) * 4; i < p.dim; i += 128) cp_async16(dst + i, src + i);
        else
          for (int i = tid & 31; i < p.dim; i += 32) cp_async4(dst + i, src + i);
      }
    asm volatile("cp.async.commit_group;\n");
  };
  auto stage_values = [&](int base, float* buf) {
    const int n = min(R, t1 - base);
    float* vs = buf + planes * R * dpad;
    for (int idx = tid; idx < n * C; idx += THREADS) {
      const int r = idx / C, c = blockIdx.x * C + idx % C;
      float v = c < p.vdim ? ld_any(p.proj, p.proj_dtype, (size_t)(base + r) * p.ld + p.v_off + (size_t)head * p.vdim + c) : 0.f;
      if (p.act == 1) v = v / (1.f + expf(-v));
      vs[idx] = v;
    }
  };

  if (p.ready) stage_async(t0, smem);
  int turn = 0;
  for (int base = t0; base < t1; base += R, turn ^= 1) {
    const int n = min(R, t1 - base);
    float* buf = smem + (p.ready ? turn : 0) * buf_floats;
    float* qs = buf;
    float* bs = buf + R * dpad;
    float* as = buf + 2 * R * dpad;
    float* vs = buf + planes * R * dpad;
    if (p.ready) {
      stage_values(base, buf);
      if (base + R < t1) {
        stage_async(base + R, smem + (turn ^ 1) * buf_floats);
        asm volatile("cp.async.wait_group 1;\n");
      } else {
        asm volatile("cp.async.wait_group 0;\n");
      }
    } else {
      for (int idx = tid; idx < n * p.dim; idx += THREADS) {
        const int r = idx / p.dim, i = idx % p.dim;
        float qv, bv, av;
        transform(p, base + r, head, i, qv, bv, av);
        qs[r * dpad + i] = qv;
        bs[r * dpad + i] = bv;
        if (gate) as[r * dpad + i] = av;
      }
      stage_values(base, buf);
    }
    __syncthreads();
    auto one_token = [&](int r) {
      const float v = vs[r * C + col_local];
      const float* qr = qs + r * dpad + slice;
      const float* br = bs + r * dpad + slice;
      float acc0 = 0.f, acc1 = 0.f;
      if (gate) {
        const float* ar = as + r * dpad + slice;
#pragma unroll
        for (int k = 0; k < ROWS; k += 2) {
          S[k] = fmaf(ar[p.slices * k], S[k], br[p.slices * k] * v);
          acc0 = fmaf(S[k], qr[p.slices * k], acc0);
          S[k + 1] = fmaf(ar[p.slices * (k + 1)], S[k + 1], br[p.slices * (k + 1)] * v);
          acc1 = fmaf(S[k + 1], qr[p.slices * (k + 1)], acc1);
        }
      } else {
#pragma unroll
        for (int k = 0; k < ROWS; k += 2) {
          S[k] = fmaf(decay, S[k], br[p.slices * k] * v);
          acc0 = fmaf(S[k], qr[p.slices * k], acc0);
          S[k + 1] = fmaf(decay, S[k + 1], br[p.slices * (k + 1)] * v);
          acc1 = fmaf(S[k + 1], qr[p.slices * (k + 1)], acc1);
        }
      }
      return acc0 + acc1;
    };
    if (n == R) {
      // a full round: the tokens' partial outputs first, then their reductions over the slices
      // side by side (the shuffles of one token do not wait for another's)
      float acc[R];
#pragma unroll
      for (int r = 0; r < R; ++r) acc[r] = one_token(r);
#pragma unroll
      for (int o = 1; o < 32; o <<= 1)
        if (o < p.slices) {
#pragma unroll
          for (int r = 0; r < R; ++r) acc[r] += __shfl_xor_sync(0xffffffffu, acc[r], o);
        }
      if (slice == 0) {
#pragma unroll
        for (int r = 0; r < R; ++r) os[r * C + col_local] = acc[r];
      }
    } else {
      for (int r = 0; r < n; ++r) {
        float acc = one_token(r);
        for (int o = 1; o < p.slices; o <<= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
        if (slice == 0) os[r * C + col_local] = acc;
      }
    }
    __syncthreads();
    for (int idx = tid; idx < n * C; idx += THREADS) {
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

template <int ROWS, int TPR>
int launch(const RecurrenceArgs& a, int S, size_t smem, cudaStream_t stream) {
  static size_t configured = 48 * 1024;
  if (smem > configured) {
    DSP_CUDA(cudaFuncSetAttribute(linear_recurrence_kernel<ROWS, TPR>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    configured = smem;
  }
  dim3 grid((a.vdim + a.cols_per_block - 1) / a.cols_per_block, a.H, S);
  linear_recurrence_kernel<ROWS, TPR><<<grid, THREADS, smem, stream>>>(a);
  DSP_CHECK_LAUNCH("dsp_linear_recurrence");
  return 0;
}
}  // namespace

// Floats of scratch the two-kernel form needs for T tokens (0: mode unknown).
extern "C" long dsp_linear_recurrence_scratch(int mode, int H, int dim, long T) {
  return (long)(mode == FORGET_GATE ? 3 : 2) * H * dim * T;
}

// scratch: null (one kernel, tokens transformed as they are staged) or room for
// dsp_linear_recurrence_scratch floats (a first kernel transforms every token, the recurrence streams).
extern "C" int dsp_linear_recurrence(const void* proj, int proj_dtype, long ld, int q_off, int k_off,
                                     int v_off, int mode, int H, int dim, int vdim, const float* decay,
                                     const float* inv_freq, int rot, float key_scale, int act,
                                     const float* gate_bias, const float* lower, float* state,
                                     const int* state_slot, const int* q_start, const int* positions,
                                     float* out, long ldo, int S, int T, float* scratch, cudaStream_t stream) {
  if (S == 0 || T == 0) return 0;
  DSP_REQUIRE(proj && state && state_slot && q_start && positions && out, "dsp_linear_recurrence: missing operand");
  DSP_REQUIRE(H > 0 && H <= 65535 && S <= 65535, "dsp_linear_recurrence: H=%d, S=%d outside the grid", H, S);
  DSP_REQUIRE(dim > 0 && dim <= 1024 && vdim > 0, "dsp_linear_recurrence: dim=%d (at most 1024), vdim=%d", dim, vdim);
  if (mode == FIXED_DECAY) {
    DSP_REQUIRE(decay != nullptr, "dsp_linear_recurrence: no decay");
    DSP_REQUIRE(rot >= 0 && rot <= dim && rot % 2 == 0 && (rot == 0 || inv_freq), "dsp_linear_recurrence: rot=%d", rot);
    DSP_REQUIRE(act == 0 || act == 1, "dsp_linear_recurrence: unknown activation %d", act);
  } else if (mode == FORGET_GATE) {
    DSP_REQUIRE(gate_bias && lower, "dsp_linear_recurrence: no gate bias or lower bound");
  } else {
    DSP_REQUIRE(false, "dsp_linear_recurrence: unknown mode %d", mode);
  }
  RecurrenceArgs a;
  a.proj = proj; a.proj_dtype = proj_dtype; a.ld = ld;
  a.q_off = q_off; a.k_off = k_off; a.v_off = v_off; a.mode = mode;
  a.H = H; a.dim = dim; a.vdim = vdim;
  a.decay = decay; a.inv_freq = inv_freq; a.rot = rot; a.key_scale = key_scale; a.act = mode == FIXED_DECAY ? act : 0;
  a.gate_bias = gate_bias; a.lower = lower;
  a.state = state; a.state_slot = state_slot; a.q_start = q_start; a.positions = positions;
  a.out = out; a.ldo = ldo; a.ready = scratch;
  // threads per column: as many as bring a thread's state rows down to 8 (a power of two, at
  // most a warp); beyond 256 rows a thread holds 16 or 32
  int slices = 1;
  while (slices < 32 && (dim + slices - 1) / slices > 8) slices *= 2;
  const int rows = (dim + slices - 1) / slices;
  a.slices = slices;
  a.cols_per_block = THREADS / slices;
  const int R = rows <= 8 ? 8 : (rows <= 16 ? 16 : 32);
  const int dpad = slices * R;
  a.tokens_per_round = dpad <= 256 ? 16 : 8;
  const int planes = mode == FORGET_GATE ? 3 : 2;
  const size_t buf = (size_t)planes * a.tokens_per_round * dpad + (size_t)a.tokens_per_round * a.cols_per_block;
  const size_t smem = sizeof(float) * ((scratch ? 2 : 1) * buf + (size_t)a.tokens_per_round * a.cols_per_block);
  if (scratch) {
    const long n = (long)T * H * dim;
    const int sms = dsp_num_sms();
    const long want = (n + 255) / 256, cap = (long)(sms > 0 ? sms : 148) * 8;
    recurrence_prepare_kernel<<<(unsigned)(want < cap ? want : cap), 256, 0, stream>>>(a, T);
    DSP_CHECK_LAUNCH("dsp_linear_recurrence (first kernel)");
  }
  if (a.tokens_per_round == 16) {
    if (R == 8) return launch<8, 16>(a, S, smem, stream);
    if (R == 16) return launch<16, 16>(a, S, smem, stream);
    return launch<32, 16>(a, S, smem, stream);
  }
  if (R == 8) return launch<8, 8>(a, S, smem, stream);
  if (R == 16) return launch<16, 8>(a, S, smem, stream);
  return launch<32, 8>(a, S, smem, stream);
}
