// Gated DeltaNet linear attention: causal depthwise conv + SiLU, gates, L2-normalised
// delta-rule state update, gated RMSNorm -- one launch per layer for 1..S tokens.
//
// Per value head h (key head hk = h / (value_heads / key_heads)) and token t:
//   c      = silu(conv4(tail, x_t))                      for the q, k and v channels
//   q, k   = c_q / sqrt(|c_q|^2 + 1e-6), c_k / sqrt(|c_k|^2 + 1e-6)
//   g      = -exp(A_log[h]) * softplus(a_t[h] + dt_bias[h]),   beta = sigmoid(b_t[h])
//   S     <- S * exp(g);  delta = (v - S^T k) * beta;  S <- S + k (x) delta
//   o      = S^T q / sqrt(key_head_dim)
//   out    = o * rsqrt(mean(o^2) + eps) * gamma * silu(z_t)
// which is the recurrence of the reference engine (cpp_engine/cuda/qwen_half_ops.cu:746-930,
// 711-730). There the steps are six kernels and the prefill form keeps a 128-float state
// column per thread; here the state tile of a head lives in registers of one block for the
// whole token run, and the projections arrive packed from one GEMM.
#include "../common/pk_common.cuh"

namespace {

using namespace pk;

constexpr int kDk = 128;  // key head dim
constexpr int kDv = 128;  // value head dim
constexpr int kThreads = 256;
constexpr int kConv = 4;

struct DeltaParams {
  const bf16* proj;    // [T, ld]: q(KD) | k(KD) | v(VD) | z(VD) | a(Hv) | b(Hv)
  int ld;
  int T;
  int key_heads, value_heads;  // local (per rank) head counts
  const float* conv_w;  // [2*KD + VD, 4], tap 3 multiplies the newest input
  float* conv_state;    // [2*KD + VD, 3], oldest first
  const float* A_log;   // [Hv]
  const float* dt_bias; // [Hv]
  const float* norm_w;  // [Dv]
  float eps;
  float* state;         // [Hv, Dk, Dv]
  bf16* out;            // [T, VD]
};

// One block per KEY head; it carries the `rep` value heads that share the key head
// (256 threads each), so q/k are convolved and normalised once and no two blocks touch
// the same conv-tail rows.
__global__ void __launch_bounds__(512) deltanet_seq_kernel(const DeltaParams p) {
  pk::pdl_wait();
  pk::pdl_trigger();
  const int hk = blockIdx.x;
  const int rep = p.value_heads / p.key_heads;
  const int KD = p.key_heads * kDk, VD = p.value_heads * kDv;
  const int tid = threadIdx.x;
  const int vh = tid >> 8;           // local value head of this thread
  const int h = hk * rep + vh;       // value head
  const int col = tid & (kDv - 1);   // value column owned by this thread
  const int half = (tid >> 7) & 1;   // which 64 rows of the key dimension
  const int nthreads = blockDim.x;

  __shared__ float s_q[kDk], s_k[kDk], s_v[4][kDv];
  __shared__ float s_part[4][2][2][kDv];  // [vh][half][kv|qv][col]
  __shared__ float s_red[40];
  __shared__ float s_gate[4][2];
  __shared__ float s_osum[4][4];

  // Conv channels of this block: q 128, k 128, v rep*128, spread over the threads in at
  // most two slots per thread.
  const int nchan = 2 * kDk + rep * kDv;
  auto chan_of = [&](int i) -> int {
    if (i < kDk) return hk * kDk + i;                       // q
    if (i < 2 * kDk) return KD + hk * kDk + (i - kDk);      // k
    return 2 * KD + hk * rep * kDv + (i - 2 * kDk);         // v (value heads are contiguous)
  };
  float cw[2][kConv], cs[2][kConv - 1];
  int cch[2];
#pragma unroll
  for (int u = 0; u < 2; ++u) {
    const int i = tid + u * nthreads;
    cch[u] = i < nchan ? chan_of(i) : -1;
    if (cch[u] >= 0) {
#pragma unroll
      for (int j = 0; j < kConv; ++j) cw[u][j] = p.conv_w[(size_t)cch[u] * kConv + j];
#pragma unroll
      for (int j = 0; j < kConv - 1; ++j) cs[u][j] = p.conv_state[(size_t)cch[u] * (kConv - 1) + j];
    }
  }

  // State tile in registers: rows [half*64, half*64+64) of column `col`.
  float S[64];
  float* sp = p.state + ((size_t)h * kDk + half * 64) * kDv + col;
#pragma unroll
  for (int i = 0; i < 64; ++i) S[i] = sp[(size_t)i * kDv];

  const float a_neg = -__expf(p.A_log[h]);
  const float dtb = p.dt_bias[h];
  const float gam = p.norm_w[col];
  const float qscale = rsqrtf((float)kDk);

  for (int t = 0; t < p.T; ++t) {
    const bf16* row = p.proj + (size_t)t * p.ld;
    // ---- conv + SiLU ----
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      if (cch[u] >= 0) {
        const float xn = __bfloat162float(row[cch[u]]);
        float y = cw[u][0] * cs[u][0] + cw[u][1] * cs[u][1] + cw[u][2] * cs[u][2] + cw[u][3] * xn;
        cs[u][0] = cs[u][1];
        cs[u][1] = cs[u][2];
        cs[u][2] = xn;
        y = silu(y);
        // Activations are 16 bit between the reference's kernels; keep that rounding.
        y = __bfloat162float(__float2bfloat16(y));
        const int i = tid + u * nthreads;
        if (i < kDk) s_q[i] = y;
        else if (i < 2 * kDk) s_k[i - kDk] = y;
        else s_v[(i - 2 * kDk) >> 7][(i - 2 * kDk) & 127] = y;
      }
    }
    if ((tid & 255) == 0) {
      const float a = __bfloat162float(row[2 * KD + 2 * VD + h]);
      const float b = __bfloat162float(row[2 * KD + 2 * VD + p.value_heads + h]);
      s_gate[vh][0] = __expf(a_neg * softplusf_(a + dtb));
      s_gate[vh][1] = sigmoidf_(b);
    }
    __syncthreads();
    // ---- L2 norms ----
    float qq = tid < kDk ? s_q[tid] * s_q[tid] : 0.f;
    float kk = tid < kDk ? s_k[tid] * s_k[tid] : 0.f;
    qq = block_sum(qq, s_red);
    kk = block_sum(kk, s_red);
    const float qn = rsqrtf(qq + 1e-6f) * qscale, kn = rsqrtf(kk + 1e-6f);
    const float decay = s_gate[vh][0], beta = s_gate[vh][1];
    // ---- S^T k and S^T q on the un-decayed state ----
    float kv = 0.f, qv = 0.f;
#pragma unroll
    for (int i = 0; i < 64; ++i) {
      const float kvv = s_k[half * 64 + i], qvv = s_q[half * 64 + i];
      kv = fmaf(S[i], kvv, kv);
      qv = fmaf(S[i], qvv, qv);
    }
    s_part[vh][half][0][col] = kv;
    s_part[vh][half][1][col] = qv;
    __syncthreads();
    kv = (s_part[vh][0][0][col] + s_part[vh][1][0][col]) * kn;
    qv = (s_part[vh][0][1][col] + s_part[vh][1][1][col]) * qn;
    float kq = 0.f;  // k . q over the whole key dim
#pragma unroll 8
    for (int i = 0; i < kDk; ++i) kq = fmaf(s_k[i], s_q[i], kq);
    kq *= kn * qn;
    const float delta = (s_v[vh][col] - decay * kv) * beta;
    const float o = decay * qv + kq * delta;
#pragma unroll
    for (int i = 0; i < 64; ++i) S[i] = fmaf(s_k[half * 64 + i] * kn, delta, S[i] * decay);
    // ---- gated RMSNorm over the head's value dim (threads with half == 0) ----
    float oo = warp_sum(half == 0 ? o * o : 0.f);
    if (half == 0 && (tid & 31) == 0) s_osum[vh][(tid >> 5) & 3] = oo;
    __syncthreads();
    if (half == 0) {
      oo = s_osum[vh][0] + s_osum[vh][1] + s_osum[vh][2] + s_osum[vh][3];
      const float z = __bfloat162float(row[2 * KD + VD + h * kDv + col]);
      const float r = rsqrtf(oo / (float)kDv + p.eps);
      p.out[(size_t)t * VD + h * kDv + col] = __float2bfloat16(o * r * gam * silu(z));
    }
    __syncthreads();
  }

#pragma unroll
  for (int i = 0; i < 64; ++i) sp[(size_t)i * kDv] = S[i];
#pragma unroll
  for (int u = 0; u < 2; ++u) {
    if (cch[u] >= 0) {
#pragma unroll
      for (int j = 0; j < kConv - 1; ++j) p.conv_state[(size_t)cch[u] * (kConv - 1) + j] = cs[u][j];
    }
  }
}

}  // namespace

// Runs tokens 0..T-1 in order, updating `state` and `conv_state` in place.
PK_API int pk_deltanet_seq(const void* proj, int ld, int T, int key_heads, int value_heads,
                           int key_dim, int value_dim, const float* conv_w, float* conv_state,
                           const float* A_log, const float* dt_bias, const float* norm_w, float eps,
                           float* state, void* out, cudaStream_t stream) {
  if (key_dim != kDk || value_dim != kDv) return PK_ERR_UNSUPPORTED;
  if (T < 1 || key_heads < 1 || value_heads < key_heads || value_heads % key_heads != 0) return PK_ERR_BAD_ARG;
  const int rep = value_heads / key_heads;
  if (rep > 2) return PK_ERR_UNSUPPORTED;  // 64 state registers per thread need <= 512 threads
  DeltaParams p{};
  p.proj = (const pk::bf16*)proj;
  p.ld = ld;
  p.T = T;
  p.key_heads = key_heads;
  p.value_heads = value_heads;
  p.conv_w = conv_w;
  p.conv_state = conv_state;
  p.A_log = A_log;
  p.dt_bias = dt_bias;
  p.norm_w = norm_w;
  p.eps = eps;
  p.state = state;
  p.out = (pk::bf16*)out;
  PK_LAUNCH_PDL(deltanet_seq_kernel, dim3(key_heads), dim3(kThreads * rep), 0, stream, p);
  return PK_OK;
}
