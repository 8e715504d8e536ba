// Gated delta rule with a decay per head and key channel, and what stands in front of it.
//
// Per head, with a state S [dim, vdim] (float32, zero at the start of a sequence, kept per slot):
//
//   S <- diag(g_t) S;   u_t = beta_t (v_t - S^T k_t);   S <- S + k_t u_t^T;   o_t = S^T q_t
//
// so the read-out sees the token's own write.  In front of it: short causal convolutions over time
// per channel of the q, k and v projections (the last taps - 1 inputs of a sequence are state too),
// SiLU, unit vectors for q and k per head (q also times dim^-1/2), beta = sigmoid(b), and the decay
// g = exp(-exp(A_log) * softplus(a + dt_bias)) per head and key channel.  All of it float32.
//
// Per-slot state, float32: [heads * dim * vdim] the matrices, then [taps - 1][channels] the
// convolutions' inputs of the last positions (channels: q, k, v as they lie in the projection).
#include "common.cuh"

#define DR_MAX_TAPS 16

__device__ __forceinline__ float dr_softplus(float z) { return z > 20.f ? z : log1pf(expf(z)); }

// One block per token.  proj [T, stride] (type T): the channels of q, k, v at q_off, k_off, v_off
// (n_qk = kv_heads * dim wide twice, n_v = heads * vdim).  conv_w: the three tap tables [channels, taps]
// one after another (q, k, v; type W).  The heads' beta pre-activations lie at b_off in proj's rows;
// a_raw [T, a_stride] float32 holds the decays' pre-activations in its first heads * dim columns.
template <typename T, typename W>
__global__ void delta_prepare_kernel(const T* __restrict__ proj, int stride, int q_off, int k_off, int v_off, int kv_heads,
                                     int heads, int dim, int vdim, int taps, const W* __restrict__ conv_w,
                                     const float* __restrict__ state, size_t state_stride, size_t tail_off,
                                     const int* __restrict__ tok_seq, const int* __restrict__ seq_start,
                                     const int* __restrict__ slots, int b_off,
                                     const float* __restrict__ a_raw, int a_stride, const W* __restrict__ dt_bias,
                                     const W* __restrict__ a_log, float q_scale, float* __restrict__ qn,
                                     float* __restrict__ kn, float* __restrict__ vc, float* __restrict__ decay,
                                     float* __restrict__ beta) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ float ch[];  // the q and k channels after convolution and SiLU
  const int t = blockIdx.x;
  const int s = tok_seq[t];
  const int r = t - seq_start[s];  // the token's place among the new tokens of its sequence
  const int n_qk = kv_heads * dim, n_v = heads * vdim, n_ch = 2 * n_qk + n_v;
  const float* tail = state + (size_t)slots[s] * state_stride + tail_off;
  for (int c = threadIdx.x; c < n_ch; c += blockDim.x) {
    const int col = c < n_qk ? q_off + c : (c < 2 * n_qk ? k_off + c - n_qk : v_off + c - 2 * n_qk);
    float acc = 0.f;
    for (int j = 0; j < taps; ++j) {
      const int back = taps - 1 - j;  // how many positions before this token the tap looks
      float xin;
      if (r - back >= 0) xin = to_f32<T>(proj[(size_t)(t - back) * stride + col]);
      else xin = tail[(size_t)(taps - 1 + r - back) * n_ch + c];
      acc = fmaf(to_f32<W>(conv_w[(size_t)c * taps + j]), xin, acc);
    }
    const float y = acc / (1.0f + expf(-acc));
    if (c < 2 * n_qk) ch[c] = y;
    else vc[(size_t)t * n_v + c - 2 * n_qk] = y;
  }
  __syncthreads();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = blockDim.x >> 5;
  for (int item = warp; item < 2 * kv_heads; item += n_warps) {  // q heads, then k heads
    const float* v = ch + (size_t)item * dim;
    float ss = 0.f;
    for (int i = lane; i < dim; i += 32) ss = fmaf(v[i], v[i], ss);
    ss = warp_sum(ss);
    const bool is_q = item < kv_heads;
    const float scale = (1.0f / sqrtf(ss + 1e-6f)) * (is_q ? q_scale : 1.0f);
    float* dst = (is_q ? qn : kn) + (size_t)t * n_qk + (size_t)(is_q ? item : item - kv_heads) * dim;
    for (int i = lane; i < dim; i += 32) dst[i] = v[i] * scale;
  }
  for (int e = threadIdx.x; e < heads * dim; e += blockDim.x) {
    const int h = e / dim;
    const float dt = dr_softplus(a_raw[(size_t)t * a_stride + e] + to_f32<W>(dt_bias[e]));
    decay[(size_t)t * heads * dim + e] = expf(-expf(to_f32<W>(a_log[h])) * dt);
  }
  for (int h = threadIdx.x; h < heads; h += blockDim.x) beta[(size_t)t * heads + h] = 1.0f / (1.0f + expf(-to_f32<T>(proj[(size_t)t * stride + b_off + h])));
}

// After the step's convolutions: the last taps - 1 inputs of every sequence, old ones kept where the
// step brought fewer.  One thread per (sequence, channel).
template <typename T>
__global__ void delta_tail_kernel(const T* __restrict__ proj, int stride, int q_off, int k_off, int v_off, int n_qk, int n_v,
                                  int taps, float* __restrict__ state, size_t state_stride, size_t tail_off,
                                  const int* __restrict__ seq_start, const int* __restrict__ slots, int n_seqs) {
  pdl_launch_dependents();
  pdl_wait();
  const int n_ch = 2 * n_qk + n_v;
  const int c = blockIdx.x * blockDim.x + threadIdx.x, s = blockIdx.y;
  if (c >= n_ch || s >= n_seqs) return;
  const int col = c < n_qk ? q_off + c : (c < 2 * n_qk ? k_off + c - n_qk : v_off + c - 2 * n_qk);
  const int start = seq_start[s], n = seq_start[s + 1] - start;
  float* tail = state + (size_t)slots[s] * state_stride + tail_off;
  float keep[DR_MAX_TAPS - 1];
#pragma unroll
  for (int j = 0; j < DR_MAX_TAPS - 1; ++j) {
    if (j < taps - 1) {
      const int src = j + n;  // place in (old tail, new inputs)
      keep[j] = src < taps - 1 ? tail[(size_t)src * n_ch + c] : to_f32<T>(proj[(size_t)(start + src - (taps - 1)) * stride + col]);
    }
  }
#pragma unroll
  for (int j = 0; j < DR_MAX_TAPS - 1; ++j)
    if (j < taps - 1) tail[(size_t)j * n_ch + c] = keep[j];
}

// The recurrence, token by token.  A block of eight warps per (sequence, head, 32 value columns): a lane
// holds its column of S in registers, a warp an eighth of the rows (RW each, a multiple of 4); the tokens' q, k
// and decay rows pass through shared memory four tokens deep (rows past dim are zeros, so that the state rows
// there stay zero and the loops need no bounds), read four numbers at a time, and one barrier per token is
// enough.  What a token needs from memory is asked for three tokens ahead and rests in registers for one token
// before it is put down, so that no load is waited for.  Since o = (gS)^T q + (k . q) u, both read-outs of the decayed state are taken in one pass over the rows.
#define DR_WARPS 8
#define DR_THREADS (DR_WARPS * 32)
template <int RW>
__global__ void __launch_bounds__(DR_THREADS) delta_rule_kernel(const float* __restrict__ qn, const float* __restrict__ kn,
                                                                const float* __restrict__ vc, const float* __restrict__ decay,
                                                                const float* __restrict__ beta, float* __restrict__ state,
                                                                size_t state_stride, const int* __restrict__ seq_start,
                                                                const int* __restrict__ slots, int heads, int kv_heads, int dim,
                                                                int vdim, int col_tiles, float* __restrict__ out) {
  pdl_launch_dependents();
  pdl_wait();
  constexpr int ROWS = DR_WARPS * RW;    // rows of the padded state, >= dim
  __shared__ __align__(16) float in[4][3][ROWS];       // [token % 4][q, k, decay][row]
  __shared__ float red[2][DR_WARPS][65];               // the warps' partial read-outs and k . q
  const int tile = blockIdx.x % col_tiles, h = (blockIdx.x / col_tiles) % heads, s = blockIdx.x / (col_tiles * heads);
  const int g = h / (heads / kv_heads);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int col = tile * 32 + lane;
  const bool live = col < vdim;
  const int row0 = warp * RW;
  const int start = seq_start[s], n = seq_start[s + 1] - start;
  float* S_g = state + (size_t)slots[s] * state_stride + (size_t)h * dim * vdim;
  float S[RW];
#pragma unroll
  for (int i = 0; i < RW; ++i) S[i] = (live && row0 + i < dim) ? S_g[(size_t)(row0 + i) * vdim + col] : 0.f;
  const int n_qk = kv_heads * dim;
  // a thread fetches at most one row of a token: ROWS <= DR_THREADS
  const int my_row = threadIdx.x;
  const bool fetches = my_row < ROWS;
  const bool in_dim = my_row < dim;
  auto fetch = [&](int tok, float& q, float& k, float& d) {
    const size_t t = (size_t)(start + tok);
    q = in_dim ? qn[t * n_qk + (size_t)g * dim + my_row] : 0.f;
    k = in_dim ? kn[t * n_qk + (size_t)g * dim + my_row] : 0.f;
    d = in_dim ? decay[(t * heads + h) * dim + my_row] : 0.f;
  };
  auto put = [&](int buf, float q, float k, float d) {
    if (fetches) { in[buf][0][my_row] = q; in[buf][1][my_row] = k; in[buf][2][my_row] = d; }
  };
  float nq = 0.f, nk = 0.f, nd = 0.f;  // the rows of token tok + 2, asked for one token ago, put down at the top of this one
  {
    float q, k, d;
    if (n > 0 && fetches) { fetch(0, q, k, d); put(0, q, k, d); }
    if (n > 1 && fetches) { fetch(1, q, k, d); put(1, q, k, d); }
    if (n > 2 && fetches) fetch(2, nq, nk, nd);
  }
  __syncthreads();
  auto v_of = [&](int tok) { return live ? vc[(size_t)(start + tok) * heads * vdim + (size_t)h * vdim + col] : 0.f; };
  auto b_of = [&](int tok) { return beta[(size_t)(start + tok) * heads + h]; };
  float v0 = n > 0 ? v_of(0) : 0.f, v1 = n > 1 ? v_of(1) : 0.f, b0 = n > 0 ? b_of(0) : 0.f, b1 = n > 1 ? b_of(1) : 0.f;
  for (int tok = 0; tok < n; ++tok) {
    const size_t t = (size_t)(start + tok);
    const int buf = tok & 3;
    const float v = v0, bt = b0;
    v0 = v1; b0 = b1;
    if (tok + 2 < n) {
      v1 = v_of(tok + 2);
      b1 = b_of(tok + 2);
      // into the buffer that token tok - 2 used: every warp has left that token by now (the barrier of tok - 1)
      put((tok + 2) & 3, nq, nk, nd);
    }
    if (tok + 3 < n && fetches) fetch(tok + 3, nq, nk, nd);
    float pk = 0.f, pq = 0.f, kq = 0.f;
    float kreg[RW];
#pragma unroll
    for (int i = 0; i < RW; i += 4) {
      const float4 q4 = *reinterpret_cast<const float4*>(&in[buf][0][row0 + i]);
      const float4 k4 = *reinterpret_cast<const float4*>(&in[buf][1][row0 + i]);
      const float4 d4 = *reinterpret_cast<const float4*>(&in[buf][2][row0 + i]);
      const float qs[4] = {q4.x, q4.y, q4.z, q4.w}, ks[4] = {k4.x, k4.y, k4.z, k4.w}, ds[4] = {d4.x, d4.y, d4.z, d4.w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float sd = S[i + e] * ds[e];
        S[i + e] = sd;
        kreg[i + e] = ks[e];
        pk = fmaf(sd, ks[e], pk);
        pq = fmaf(sd, qs[e], pq);
        kq = fmaf(ks[e], qs[e], kq);
      }
    }
    float* rd = &red[tok & 1][0][0];
    rd[warp * 65 + lane] = pk;
    rd[warp * 65 + 32 + lane] = pq;
    if (lane == 0) rd[warp * 65 + 64] = kq;
    __syncthreads();
    float sk = 0.f, sq = 0.f, skq = 0.f;
#pragma unroll
    for (int w = 0; w < DR_WARPS; ++w) {
      sk += rd[w * 65 + lane];
      sq += rd[w * 65 + 32 + lane];
      skq += rd[w * 65 + 64];
    }
    const float u = bt * (v - sk);
#pragma unroll
    for (int i = 0; i < RW; ++i) S[i] = fmaf(kreg[i], u, S[i]);
    if (warp == 0 && live) out[t * heads * vdim + (size_t)h * vdim + col] = fmaf(skq, u, sq);
  }
  if (live) {
#pragma unroll
    for (int i = 0; i < RW; ++i)
      if (row0 + i < dim) S_g[(size_t)(row0 + i) * vdim + col] = S[i];
  }
}

static int dr_types(int dtype, int w_dtype) {
  if ((dtype != BN_F32 && dtype != BN_BF16) || (w_dtype != BN_F32 && w_dtype != BN_BF16)) return -1;
  return dtype * 2 + w_dtype;
}

// See the kernels above.  state [slots, state_stride] float32 with the convolutions' inputs from tail_off on.
extern "C" int bn_delta_prepare(const void* proj, int dtype, int n_tokens, int stride, int q_off, int k_off, int v_off,
                                int kv_heads, int heads, int dim, int vdim, int taps, const void* conv_w, int w_dtype,
                                float* state, long long state_stride, long long tail_off, const int* tok_seq,
                                const int* seq_start, const int* slots, int n_seqs, int b_off, const float* a_raw, int a_stride,
                                const void* dt_bias, const void* a_log, float q_scale, float* qn, float* kn, float* vc,
                                float* decay, float* beta, cudaStream_t stream) {
  if (n_tokens <= 0) return BN_OK;
  const int n_qk = kv_heads * dim, n_v = heads * vdim;
  if (kv_heads <= 0 || heads % kv_heads || dim <= 0 || vdim <= 0 || taps < 1 || taps > DR_MAX_TAPS || !proj || !conv_w ||
      !state || !tok_seq || !seq_start || !slots || b_off < 0 || b_off + heads > stride || !a_raw || a_stride < heads * dim || !dt_bias || !a_log || !qn || !kn || !vc || !decay ||
      !beta || q_off < 0 || k_off < 0 || v_off < 0 || q_off + n_qk > stride || k_off + n_qk > stride || v_off + n_v > stride ||
      (size_t)2 * n_qk * sizeof(float) > 160 * 1024)
    return BN_ERR_BAD_ARG;
  const size_t smem = (size_t)2 * n_qk * sizeof(float);
#define DR_PREP(TT, WW)                                                                                                    \
  do {                                                                                                                     \
    if (smem > 48 * 1024) {                                                                                                \
      static size_t granted = 0;                                                                                           \
      if (smem > granted) {                                                                                                \
        cudaError_t e = cudaFuncSetAttribute(delta_prepare_kernel<TT, WW>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        if (e != cudaSuccess) return BN_ERR_LAUNCH + (int)e;                                                               \
        granted = smem;                                                                                                    \
      }                                                                                                                    \
    }                                                                                                                      \
    BN_LAUNCH((delta_prepare_kernel<TT, WW>), n_tokens, 256, smem, stream, (const TT*)proj, stride, q_off, k_off, v_off,  \
              kv_heads, heads, dim, vdim, taps, (const WW*)conv_w, (const float*)state, (size_t)state_stride,             \
              (size_t)tail_off, tok_seq, seq_start, slots, b_off, a_raw, a_stride, (const WW*)dt_bias, (const WW*)a_log, q_scale,   \
              qn, kn, vc, decay, beta);                                                                                    \
  } while (0)
  switch (dr_types(dtype, w_dtype)) {
    case 0: DR_PREP(float, float); break;
    case 2: DR_PREP(__nv_bfloat16, float); break;
    case 3: DR_PREP(__nv_bfloat16, __nv_bfloat16); break;
    default: return BN_ERR_BAD_ARG;
  }
#undef DR_PREP
  if (taps > 1) {
    dim3 grid((2 * n_qk + n_v + 255) / 256, n_seqs);
    if (dtype == BN_F32)
      BN_LAUNCH(delta_tail_kernel<float>, grid, 256, 0, stream, (const float*)proj, stride, q_off, k_off, v_off, n_qk, n_v,
                taps, state, (size_t)state_stride, (size_t)tail_off, seq_start, slots, n_seqs);
    else
      BN_LAUNCH(delta_tail_kernel<__nv_bfloat16>, grid, 256, 0, stream, (const __nv_bfloat16*)proj, stride, q_off, k_off,
                v_off, n_qk, n_v, taps, state, (size_t)state_stride, (size_t)tail_off, seq_start, slots, n_seqs);
  }
  return BN_OK;
}

// qn, kn [T, kv_heads * dim], vc [T, heads * vdim], decay [T, heads * dim], beta [T, heads], all float32 as
// bn_delta_prepare leaves them; out [T, heads * vdim] float32; dim up to 256.
extern "C" int bn_delta_rule(const float* qn, const float* kn, const float* vc, const float* decay, const float* beta,
                             float* state, long long state_stride, const int* seq_start, const int* slots, int n_seqs,
                             int heads, int kv_heads, int dim, int vdim, float* out, cudaStream_t stream) {
  if (n_seqs <= 0) return BN_OK;
  if (!qn || !kn || !vc || !decay || !beta || !state || !seq_start || !slots || !out || kv_heads <= 0 || heads % kv_heads ||
      dim <= 0 || dim > 256 || vdim <= 0)
    return BN_ERR_BAD_ARG;
  const int col_tiles = (vdim + 31) / 32;
  const long long blocks = (long long)n_seqs * heads * col_tiles;
  if (blocks > 2147483647LL) return BN_ERR_BAD_ARG;
#define DR_RUN(RW)                                                                                                      \
  BN_LAUNCH(delta_rule_kernel<RW>, (unsigned)blocks, DR_THREADS, 0, stream, qn, kn, vc, decay, beta, state, (size_t)state_stride, \
            seq_start, slots, heads, kv_heads, dim, vdim, col_tiles, out)
  if (dim <= 32) DR_RUN(4);
  else if (dim <= 64) DR_RUN(8);
  else if (dim <= 128) DR_RUN(16);
  else DR_RUN(32);
#undef DR_RUN
  return BN_OK;
}

// Behind the recurrence: each head's o divided by its root mean square over vdim (eps), times a gain
// [vdim] that all heads share, times the logistic function of a float32 gate (row stride gate_stride).
// One warp per (token, head).
template <typename T, typename W>
__global__ void delta_output_kernel(const float* __restrict__ o, const W* __restrict__ gain, const float* __restrict__ gate,
                                    int gate_stride, int heads, int vdim, float eps, T* __restrict__ out, int n_items) {
  pdl_launch_dependents();
  pdl_wait();
  const int item = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (item >= n_items) return;
  const int t = item / heads, h = item - t * heads;
  const float* oh = o + (size_t)item * vdim;
  float ss = 0.f;
  for (int c = lane; c < vdim; c += 32) ss = fmaf(oh[c], oh[c], ss);
  ss = warp_sum(ss);
  const float scale = 1.0f / sqrtf(ss / (float)vdim + eps);
  for (int c = lane; c < vdim; c += 32) {
    const float gt = 1.0f / (1.0f + expf(-gate[(size_t)t * gate_stride + (size_t)h * vdim + c]));
    out[(size_t)item * vdim + c] = from_f32<T>(oh[c] * scale * to_f32<W>(gain[c]) * gt);
  }
}

extern "C" int bn_delta_output(const float* o, const void* gain, int gain_dtype, const float* gate, int gate_stride, int dtype,
                               int n_tokens, int heads, int vdim, float eps, void* out, cudaStream_t stream) {
  if (n_tokens <= 0) return BN_OK;
  if (!o || !gain || !gate || !out || heads <= 0 || vdim <= 0 || gate_stride < heads * vdim || !(eps > 0.f)) return BN_ERR_BAD_ARG;
  const int items = n_tokens * heads;
  const unsigned blocks = (unsigned)((items + 7) / 8);
  switch (dr_types(dtype, gain_dtype)) {
    case 0: BN_LAUNCH((delta_output_kernel<float, float>), blocks, 256, 0, stream, o, (const float*)gain, gate, gate_stride, heads, vdim, eps, (float*)out, items); break;
    case 2: BN_LAUNCH((delta_output_kernel<__nv_bfloat16, float>), blocks, 256, 0, stream, o, (const float*)gain, gate, gate_stride, heads, vdim, eps, (__nv_bfloat16*)out, items); break;
    case 3: BN_LAUNCH((delta_output_kernel<__nv_bfloat16, __nv_bfloat16>), blocks, 256, 0, stream, o, (const __nv_bfloat16*)gain, gate, gate_stride, heads, vdim, eps, (__nv_bfloat16*)out, items); break;
    default: return BN_ERR_BAD_ARG;
  }
  return BN_OK;
}
