// mLSTM: a matrix memory per head with exponential input gate and a stabiliser.
//
// Per head, with log input gate i_t, log forget gate f_t (both float32), keys k_t and queries q_t of
// `dim` numbers (the query already scaled) and values v_t of `vdim` numbers:
//
//   m_t = max(f_t + m_{t-1}, i_t)
//   a = exp(f_t + m_{t-1} - m_t),  b = exp(i_t - m_t)
//   S_t = a S_{t-1} + b k_t v_t^T          [dim, vdim]
//   n_t = a n_{t-1} + b k_t                [dim]
//   o_t = S_t^T q_t / (max(|n_t . q_t|, exp(-m_t)) + 1e-6)
//
// S, n and m start at zero for a new sequence and live in float32 in the state manager's tensor
//   state[slot][head] = { S[dim][vdim], n[dim], m }
// from step to step.  The three kernels here:
//   bn_mlstm_gates       i, f from the mixer's input (a float32 product with 2 * heads rows) with their soft cap
//   bn_mlstm_recurrence  the recurrence over the new tokens of every sequence, token by token
//   bn_mlstm_output      per head o / rms(o), times a gain over all heads, times the logistic output gate
#include "common.cuh"

#define ML_GATE_THREADS 128

// gates[t][0..H) = cap * tanh((W_i h + b_i) / cap);  gates[t][H..2H) = logsigmoid(cap * tanh((W_f h + b_f) / cap))
// w: [2H, width] (input gate rows first), bias: [2H].
template <typename T, typename W>
__global__ void mlstm_gates_kernel(const T* __restrict__ h, int width, const W* __restrict__ w,
                                   const W* __restrict__ bias, int n_heads, float cap, float* __restrict__ gates) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ __align__(16) float xs[];  // width
  const int t = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = blockDim.x >> 5;
  const T* row = h + (size_t)t * width;
  for (int c = threadIdx.x; c < width; c += blockDim.x) xs[c] = to_f32<T>(row[c]);
  __syncthreads();
  for (int r = warp; r < 2 * n_heads; r += n_warps) {
    float dot = warp_dot(xs, w + (size_t)r * width, width, lane);
    if (lane == 0) {
      float z = cap * tanhf((dot + to_f32<W>(bias[r])) / cap);
      if (r >= n_heads) z = fminf(z, 0.f) - log1pf(expf(-fabsf(z)));  // log(sigmoid(z))
      gates[(size_t)t * 2 * n_heads + r] = z;
    }
  }
}

extern "C" int bn_mlstm_gates(const void* h, int h_dtype, int n_tokens, int width, const void* w, const void* bias,
                              int w_dtype, int n_heads, float cap, float* gates, cudaStream_t stream) {
  if (n_tokens <= 0) return BN_OK;
  if (!h || !w || !bias || !gates || width <= 0 || n_heads <= 0 || !(cap > 0.f) || (size_t)width * sizeof(float) > 48 * 1024)
    return BN_ERR_BAD_ARG;
  const size_t smem = (size_t)width * sizeof(float);
  if (h_dtype == BN_F32 && w_dtype == BN_F32)
    BN_LAUNCH((mlstm_gates_kernel<float, float>), n_tokens, ML_GATE_THREADS, smem, stream, (const float*)h, width,
              (const float*)w, (const float*)bias, n_heads, cap, gates);
  else if (h_dtype == BN_BF16 && w_dtype == BN_BF16)
    BN_LAUNCH((mlstm_gates_kernel<__nv_bfloat16, __nv_bfloat16>), n_tokens, ML_GATE_THREADS, smem, stream,
              (const __nv_bfloat16*)h, width, (const __nv_bfloat16*)w, (const __nv_bfloat16*)bias, n_heads, cap, gates);
  else if (h_dtype == BN_BF16 && w_dtype == BN_F32)
    BN_LAUNCH((mlstm_gates_kernel<__nv_bfloat16, float>), n_tokens, ML_GATE_THREADS, smem, stream,
              (const __nv_bfloat16*)h, width, (const float*)w, (const float*)bias, n_heads, cap, gates);
  else
    return BN_ERR_BAD_ARG;
  BN_CHECK_LAUNCH();
  return BN_OK;
}

// One block per (sequence, head, chunk of value columns); thread c owns column c0 + c of S, which
// lies in shared memory as S[d][c].  Every block of a head keeps n and m itself (the same numbers
// in the same order in each), the block of chunk 0 writes them back.
template <typename T>
__global__ void mlstm_recurrence_kernel(const T* __restrict__ qkv, int row_stride, int k_off, int v_off,
                                        const float* __restrict__ gates, float* __restrict__ state,
                                        const int* __restrict__ seq_start, const int* __restrict__ slots, int n_heads,
                                        int dim, int vdim, int cols, float q_scale, float* __restrict__ out) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ float sm[];
  float* S = sm;                   // dim * cols
  float* sq = S + (size_t)dim * cols;  // dim
  float* sk = sq + dim;            // dim
  float* sn = sk + dim;            // dim
  const int seq = blockIdx.x, head = blockIdx.y, c0 = blockIdx.z * cols;
  const int c = threadIdx.x, lane = threadIdx.x & 31;
  const bool has_col = c < cols && c0 + c < vdim;
  const size_t per_head = (size_t)dim * vdim + dim + 1;
  float* st = state + ((size_t)slots[seq] * n_heads + head) * per_head;
  float* st_n = st + (size_t)dim * vdim;
  if (has_col)
    for (int d = 0; d < dim; ++d) S[d * cols + c] = st[(size_t)d * vdim + c0 + c];
  for (int d = threadIdx.x; d < dim; d += blockDim.x) sn[d] = st_n[d];
  float m = st_n[dim];
  const int t0 = seq_start[seq], t1 = seq_start[seq + 1];
  for (int t = t0; t < t1; ++t) {
    const T* row = qkv + (size_t)t * row_stride;
    __syncthreads();  // the step before has read sq, sk
    for (int d = threadIdx.x; d < dim; d += blockDim.x) {
      sq[d] = to_f32<T>(row[(size_t)head * dim + d]) * q_scale;
      sk[d] = to_f32<T>(row[k_off + (size_t)head * dim + d]);
    }
    float gi = gates[(size_t)t * 2 * n_heads + head], gf = gates[(size_t)t * 2 * n_heads + n_heads + head];
    float m_new = fmaxf(gf + m, gi);
    float a = expf(gf + m - m_new), b = expf(gi - m_new);
    m = m_new;
    __syncthreads();
    for (int d = threadIdx.x; d < dim; d += blockDim.x) sn[d] = a * sn[d] + b * sk[d];
    __syncthreads();
    float nq = 0.f;
    for (int d = lane; d < dim; d += 32) nq = fmaf(sn[d], sq[d], nq);
    nq = warp_sum(nq);
    float denom = fmaxf(fabsf(nq), expf(-m)) + 1e-6f;
    if (has_col) {
      float v = to_f32<T>(row[v_off + (size_t)head * vdim + c0 + c]);
      float bv = b * v, acc = 0.f;
      for (int d = 0; d < dim; ++d) {
        float s = fmaf(a, S[d * cols + c], bv * sk[d]);
        S[d * cols + c] = s;
        acc = fmaf(s, sq[d], acc);
      }
      out[(size_t)t * n_heads * vdim + (size_t)head * vdim + c0 + c] = acc / denom;
    }
  }
  if (has_col)
    for (int d = 0; d < dim; ++d) st[(size_t)d * vdim + c0 + c] = S[d * cols + c];
  __syncthreads();
  if (blockIdx.z == 0) {
    for (int d = threadIdx.x; d < dim; d += blockDim.x) st_n[d] = sn[d];
    if (threadIdx.x == 0) st_n[dim] = m;
  }
}

// Head sizes up to 128: a block of four warps per (sequence, head, 32 value columns).  Each warp keeps a
// quarter of the rows of S for the block's 32 columns in registers (one column per lane, D / 4 rows, dim
// padded with zeros to D), its rows' share of n spread over its lanes, and hands its rows of q and k
// round through shared memory of its own.  Per token the warps' partial sums of S^T q and n . q meet in
// shared memory behind one barrier (two sets of buffers in turn); warp 0 adds them, always in the same
// order, and stores.  The next token's row is requested while this one's is worked on.
template <typename T, int D>
__global__ void __launch_bounds__(128) mlstm_recurrence_warp_kernel(
    const T* __restrict__ qkv, int row_stride, int k_off, int v_off, const float* __restrict__ gates,
    float* __restrict__ state, const int* __restrict__ seq_start, const int* __restrict__ slots, int n_heads, int dim,
    int vdim, float q_scale, float* __restrict__ out) {
  pdl_launch_dependents();
  pdl_wait();
  constexpr int DW = D / 4;  // rows of S per warp: 8, 16 or 32
  __shared__ __align__(16) float sq[4][DW], sk[4][DW];
  __shared__ float part_o[2][4][32], part_nq[2][4];
  const int seq = blockIdx.x, head = blockIdx.y, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int c = blockIdx.z * 32 + lane;
  const bool has_col = c < vdim;
  const int d0 = warp * DW;           // this warp's first row
  const int my_d = d0 + lane;         // the row whose q, k and n this lane holds (lanes below DW)
  const bool has_row = lane < DW && my_d < dim;
  const size_t per_head = (size_t)dim * vdim + dim + 1;
  float* st = state + ((size_t)slots[seq] * n_heads + head) * per_head;
  float* st_n = st + (size_t)dim * vdim;
  float S[DW];
#pragma unroll
  for (int r = 0; r < DW; ++r) S[r] = (has_col && d0 + r < dim) ? st[(size_t)(d0 + r) * vdim + c] : 0.f;
  float n = has_row ? st_n[my_d] : 0.f;
  float m = st_n[dim];
  const int t0 = seq_start[seq], t1 = seq_start[seq + 1];
  float qn = 0.f, kn = 0.f, vn = 0.f, gi_n = 0.f, gf_n = 0.f;
  auto fetch = [&](int t) {
    const T* row = qkv + (size_t)t * row_stride;
    qn = has_row ? to_f32<T>(row[(size_t)head * dim + my_d]) * q_scale : 0.f;
    kn = has_row ? to_f32<T>(row[k_off + (size_t)head * dim + my_d]) : 0.f;
    vn = has_col ? to_f32<T>(row[v_off + (size_t)head * vdim + c]) : 0.f;
    gi_n = gates[(size_t)t * 2 * n_heads + head];
    gf_n = gates[(size_t)t * 2 * n_heads + n_heads + head];
  };
  if (t0 < t1) fetch(t0);
  for (int t = t0; t < t1; ++t) {
    const float q = qn, k = kn, v = vn, gi = gi_n, gf = gf_n;
    const int buf = (t - t0) & 1;
    __syncwarp();  // the step before has read this warp's sq, sk
    if (lane < DW) { sq[warp][lane] = q; sk[warp][lane] = k; }
    if (t + 1 < t1) fetch(t + 1);
    float m_new = fmaxf(gf + m, gi);
    float a = expf(gf + m - m_new), b = expf(gi - m_new);
    m = m_new;
    n = a * n + b * k;
    float nq = warp_sum(n * q);
    __syncwarp();
    float bv = b * v, acc0 = 0.f, acc1 = 0.f, acc2 = 0.f, acc3 = 0.f;
#pragma unroll
    for (int r = 0; r < DW; r += 4) {
      float4 k4 = *reinterpret_cast<const float4*>(&sk[warp][r]), q4 = *reinterpret_cast<const float4*>(&sq[warp][r]);
      S[r] = fmaf(a, S[r], bv * k4.x);         acc0 = fmaf(S[r], q4.x, acc0);
      S[r + 1] = fmaf(a, S[r + 1], bv * k4.y); acc1 = fmaf(S[r + 1], q4.y, acc1);
      S[r + 2] = fmaf(a, S[r + 2], bv * k4.z); acc2 = fmaf(S[r + 2], q4.z, acc2);
      S[r + 3] = fmaf(a, S[r + 3], bv * k4.w); acc3 = fmaf(S[r + 3], q4.w, acc3);
    }
    part_o[buf][warp][lane] = (acc0 + acc1) + (acc2 + acc3);
    if (lane == 0) part_nq[buf][warp] = nq;
    __syncthreads();
    if (warp == 0) {
      float o = (part_o[buf][0][lane] + part_o[buf][1][lane]) + (part_o[buf][2][lane] + part_o[buf][3][lane]);
      float nq_all = (part_nq[buf][0] + part_nq[buf][1]) + (part_nq[buf][2] + part_nq[buf][3]);
      float denom = fmaxf(fabsf(nq_all), expf(-m)) + 1e-6f;
      if (has_col) out[(size_t)t * n_heads * vdim + (size_t)head * vdim + c] = o / denom;
    }
  }
  if (has_col) {
#pragma unroll
    for (int r = 0; r < DW; ++r)
      if (d0 + r < dim) st[(size_t)(d0 + r) * vdim + c] = S[r];
  }
  if (blockIdx.z == 0) {
    if (has_row) st_n[my_d] = n;
    if (threadIdx.x == 0) st_n[dim] = m;
  }
}

template <typename T>
static cudaError_t launch_mlstm_warp(const void* qkv, int row_stride, int k_off, int v_off, const float* gates, float* state,
                                     const int* seq_start, const int* slots, int n_seqs, int n_heads, int dim, int vdim,
                                     float q_scale, float* out, cudaStream_t stream) {
  dim3 grid(n_seqs, n_heads, (vdim + 31) / 32);
  if (dim <= 32)
    return bn_launch(mlstm_recurrence_warp_kernel<T, 32>, grid, dim3(128), 0, stream, (const T*)qkv, row_stride, k_off, v_off,
                     gates, state, seq_start, slots, n_heads, dim, vdim, q_scale, out);
  if (dim <= 64)
    return bn_launch(mlstm_recurrence_warp_kernel<T, 64>, grid, dim3(128), 0, stream, (const T*)qkv, row_stride, k_off, v_off,
                     gates, state, seq_start, slots, n_heads, dim, vdim, q_scale, out);
  return bn_launch(mlstm_recurrence_warp_kernel<T, 128>, grid, dim3(128), 0, stream, (const T*)qkv, row_stride, k_off, v_off,
                   gates, state, seq_start, slots, n_heads, dim, vdim, q_scale, out);
}

// qkv: rows of the new tokens with the query heads at element 0, key heads at k_off, value heads at
// v_off; gates [n_tokens, 2 * heads]; state [slots, heads, dim * vdim + dim + 1]; out [n_tokens, heads * vdim] float32.
extern "C" int bn_mlstm_recurrence(const void* qkv, int dtype, int row_stride, int k_off, int v_off, const float* gates,
                                   float* state, const int* seq_start, const int* slots, int n_seqs, int n_heads, int dim,
                                   int vdim, float q_scale, float* out, cudaStream_t stream) {
  if (n_seqs <= 0) return BN_OK;
  if (!qkv || !gates || !state || !out || n_heads <= 0 || dim <= 0 || vdim <= 0 || n_heads > 65535) return BN_ERR_BAD_ARG;
  if (dim <= 128 && (vdim + 31) / 32 <= 65535 && (dtype == BN_F32 || dtype == BN_BF16)) {
    cudaError_t e = dtype == BN_F32
        ? launch_mlstm_warp<float>(qkv, row_stride, k_off, v_off, gates, state, seq_start, slots, n_seqs, n_heads, dim, vdim,
                                   q_scale, out, stream)
        : launch_mlstm_warp<__nv_bfloat16>(qkv, row_stride, k_off, v_off, gates, state, seq_start, slots, n_seqs, n_heads, dim,
                                           vdim, q_scale, out, stream);
    if (e != cudaSuccess) return BN_ERR_LAUNCH + (int)e;
    BN_CHECK_LAUNCH();
    return BN_OK;
  }
  int cols = vdim >= 128 ? 128 : (vdim + 31) / 32 * 32;
  while (cols > 32 && ((size_t)dim * cols + 3 * dim) * sizeof(float) > 160 * 1024) cols /= 2;
  size_t smem = ((size_t)dim * cols + 3 * (size_t)dim) * sizeof(float);
  if (smem > 200 * 1024) return BN_ERR_BAD_ARG;
  int chunks = (vdim + cols - 1) / cols;
  if (chunks > 65535) return BN_ERR_BAD_ARG;
  dim3 grid(n_seqs, n_heads, chunks);
  static size_t granted_f = 0, granted_b = 0;
  if (dtype == BN_F32) {
    if (smem > 48 * 1024 && smem > granted_f) {
      cudaError_t e = cudaFuncSetAttribute(mlstm_recurrence_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (e != cudaSuccess) return BN_ERR_LAUNCH + (int)e;
      granted_f = smem;
    }
    BN_LAUNCH(mlstm_recurrence_kernel<float>, grid, cols, smem, stream, (const float*)qkv, row_stride, k_off, v_off, gates,
              state, seq_start, slots, n_heads, dim, vdim, cols, q_scale, out);
  } else if (dtype == BN_BF16) {
    if (smem > 48 * 1024 && smem > granted_b) {
      cudaError_t e = cudaFuncSetAttribute(mlstm_recurrence_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (e != cudaSuccess) return BN_ERR_LAUNCH + (int)e;
      granted_b = smem;
    }
    BN_LAUNCH(mlstm_recurrence_kernel<__nv_bfloat16>, grid, cols, smem, stream, (const __nv_bfloat16*)qkv, row_stride,
              k_off, v_off, gates, state, seq_start, slots, n_heads, dim, vdim, cols, q_scale, out);
  } else {
    return BN_ERR_BAD_ARG;
  }
  BN_CHECK_LAUNCH();
  return BN_OK;
}

// ---- runs of many tokens: the recurrence chunk by chunk ------------------------------------------
// Within a chunk of 32 tokens the recurrence is unrolled into sums.  With F_t the sum of the forget
// gates from the chunk's first token to t, z_s = i_s - F_s and M_t = max(m0, max_{s<=t} z_s)
// (m0: the stabiliser before the chunk), the stabiliser after token t is m_t = F_t + M_t, and
//
//   S_t = sum_{s<=t} e^{z_s - M_t} k_s v_s^T + e^{m0 - M_t} S0        (every exponent is <= 0)
//
// so  S_t^T q_t = sum_{s<=t} e^{z_s - M_t} (q_t . k_s) v_s + e^{m0 - M_t} S0^T q_t, likewise n_t . q_t with
// the v_s left out, and the state after the chunk is S_t, n_t, m_t at its last token.  Per chunk that is
// four small matrix products in float32 (Q K^T, P V, Q S0, K^T V) instead of 32 dependent steps; the
// chunks of a sequence follow one another through the state.  One block of 128 threads per (sequence,
// head, 32 value columns); the 32 tokens of a chunk are the 32 lanes of a warp for the scans.
// The sums run in another order than token by token, so the two forms agree to rounding, not bit by bit.
#define MLC_L 32
#define MLC_THREADS 512
#define MLC_ROWS (MLC_L / (MLC_THREADS / 32))  // rows of a chunk per warp

template <typename T>
__global__ void __launch_bounds__(MLC_THREADS) mlstm_chunk_kernel(
    const T* __restrict__ qkv, int row_stride, int k_off, int v_off, const float* __restrict__ gates,
    float* __restrict__ state, const int* __restrict__ seq_start, const int* __restrict__ slots, int n_heads, int dim,
    int vdim, float q_scale, float* __restrict__ out) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ __align__(16) float sm[];
  const int ld = dim + 4;                 // padded rows of Q and K
  float* sQ = sm;                         // [L][ld]
  float* sK = sQ + MLC_L * ld;            // [L][ld]
  float* sS = sK + MLC_L * ld;            // [dim][32]
  float* sV = sS + (size_t)dim * 32;      // [L][32]
  float* sP = sV + MLC_L * 32;            // [L][L + 1]
  float* sn = sP + MLC_L * (MLC_L + 1);   // [dim]
  float* s_nq = sn + dim;                 // [L]
  float* s_g = s_nq + MLC_L;              // [L]: each token's weight in the state after the chunk
  const int seq = blockIdx.x, head = blockIdx.y, c0 = blockIdx.z * 32;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int c = c0 + lane;
  const bool has_col = c < vdim;
  const size_t per_head = (size_t)dim * vdim + dim + 1;
  float* st = state + ((size_t)slots[seq] * n_heads + head) * per_head;
  float* st_n = st + (size_t)dim * vdim;
  for (int i = tid; i < dim * 32; i += MLC_THREADS) {
    int d = i >> 5, cc = i & 31;
    sS[i] = (c0 + cc < vdim) ? st[(size_t)d * vdim + c0 + cc] : 0.f;
  }
  for (int d = tid; d < dim; d += MLC_THREADS) sn[d] = st_n[d];
  float m0 = st_n[dim];
  const int t0 = seq_start[seq], t1 = seq_start[seq + 1];
  // Rows of whole 16-byte pieces (the usual case) are read in such pieces, and a chunk's q and k rows are
  // requested into registers while the chunk before is worked on; other sizes go number by number.
  constexpr int VN = 16 / sizeof(T);
  constexpr int MAXV = 2;  // pieces per thread and matrix: 32 rows of up to 128 numbers in float32, 256 in bfloat16
  const bool wide = dim % VN == 0 && k_off % VN == 0 && row_stride % VN == 0 && v_off % VN == 0 && vdim % VN == 0 &&
                    (((uintptr_t)qkv) & 15) == 0 && MLC_L * dim / VN <= MAXV * MLC_THREADS;
  const int pieces = wide ? MLC_L * dim / VN : 0, per_row = wide ? dim / VN : 1;
  uint4 rq[MAXV], rk[MAXV];
  auto request = [&](int base) {
    const int n_tok = min(MLC_L, t1 - base);
#pragma unroll
    for (int j = 0; j < MAXV; ++j) {
      int idx = tid + j * MLC_THREADS;
      int t = idx / per_row, d = (idx - t * per_row) * VN;
      if (idx < pieces && t < n_tok) {
        const T* row = qkv + (size_t)(base + t) * row_stride + (size_t)head * dim + d;
        rq[j] = *reinterpret_cast<const uint4*>(row);
        rk[j] = *reinterpret_cast<const uint4*>(row + k_off);
      } else {
        rq[j] = make_uint4(0, 0, 0, 0);
        rk[j] = make_uint4(0, 0, 0, 0);
      }
    }
  };
  auto unpack = [&](const uint4& raw, float* dst, float scale) {  // dst is 16-byte aligned
    const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
    for (int i = 0; i < VN; i += 4)
      *reinterpret_cast<float4*>(dst + i) = make_float4(to_f32<T>(e[i]) * scale, to_f32<T>(e[i + 1]) * scale,
                                                        to_f32<T>(e[i + 2]) * scale, to_f32<T>(e[i + 3]) * scale);
  };
  if (wide && t0 < t1) request(t0);
  for (int base = t0; base < t1; base += MLC_L) {
    const int n_tok = min(MLC_L, t1 - base);
    __syncthreads();  // the chunk before is done with sQ, sK, sV, sP; sS and sn are up to date
    if (wide) {
#pragma unroll
      for (int j = 0; j < MAXV; ++j) {
        int idx = tid + j * MLC_THREADS;
        if (idx < pieces) {
          int t = idx / per_row, d = (idx - t * per_row) * VN;
          unpack(rq[j], sQ + t * ld + d, q_scale);
          unpack(rk[j], sK + t * ld + d, 1.0f);
        }
      }
      if (base + MLC_L < t1) request(base + MLC_L);
    } else {
      for (int i = tid; i < MLC_L * dim; i += MLC_THREADS) {
        int t = i / dim, d = i - t * dim;
        bool ok = t < n_tok;
        const T* row = qkv + (size_t)(base + t) * row_stride;
        sQ[t * ld + d] = ok ? to_f32<T>(row[(size_t)head * dim + d]) * q_scale : 0.f;
        sK[t * ld + d] = ok ? to_f32<T>(row[k_off + (size_t)head * dim + d]) : 0.f;
      }
    }
    if (wide && c0 + 32 <= vdim) {
      for (int idx = tid; idx < MLC_L * 32 / VN; idx += MLC_THREADS) {
        int t = idx / (32 / VN), cc = (idx - t * (32 / VN)) * VN;
        uint4 raw = make_uint4(0, 0, 0, 0);
        if (t < n_tok) raw = *reinterpret_cast<const uint4*>(qkv + (size_t)(base + t) * row_stride + v_off + (size_t)head * vdim + c0 + cc);
        unpack(raw, sV + t * 32 + cc, 1.0f);
      }
    } else {
      for (int i = tid; i < MLC_L * 32; i += MLC_THREADS) {
        int t = i >> 5, cc = i & 31;
        sV[i] = (t < n_tok && c0 + cc < vdim) ? to_f32<T>(qkv[(size_t)(base + t) * row_stride + v_off + (size_t)head * vdim + c0 + cc]) : 0.f;
      }
    }
    // the chunk's scalars, in every warp alike: lane = token
    const bool valid = lane < n_tok;
    float gi = valid ? gates[(size_t)(base + lane) * 2 * n_heads + head] : 0.f;
    float gf = valid ? gates[(size_t)(base + lane) * 2 * n_heads + n_heads + head] : 0.f;
    float F = gf;  // inclusive sum over the lanes
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      float up = __shfl_up_sync(0xffffffffu, F, o);
      if (lane >= o) F += up;
    }
    float z = valid ? gi - F : -INFINITY;
    float G = z;   // inclusive maximum over the lanes
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      float up = __shfl_up_sync(0xffffffffu, G, o);
      if (lane >= o) G = fmaxf(G, up);
    }
    const float M = fmaxf(m0, G);          // M_t of this lane's token
    const float carry = expf(m0 - M);      // weight of the state before the chunk at this token
    const float m_tok = F + M;             // the stabiliser after this token
    const float M_last = __shfl_sync(0xffffffffu, M, n_tok - 1);
    const float g_state = valid ? expf(z - M_last) : 0.f;  // weight of this token in the state after the chunk
    const float carry_last = expf(m0 - M_last);
    const float m_end = __shfl_sync(0xffffffffu, m_tok, n_tok - 1);
    if (warp == 0) s_g[lane] = g_state;
    __syncthreads();  // sQ, sK, sV, s_g are loaded
    // ---- P[t][s] = (q_t . k_s) e^{z_s - M_t} for s <= t: thread = (row t, columns s = s0 + TPR j), so that
    // the threads of a row read neighbouring rows of K (rows lie dim + 4 numbers apart: no two in one bank)
    {
      constexpr int TPR = MLC_THREADS / MLC_L;  // threads per row
      constexpr int CPT = MLC_L / TPR;          // columns per thread
      const int t = tid / TPR, s0 = tid % TPR;
      float acc[CPT];
#pragma unroll
      for (int j = 0; j < CPT; ++j) acc[j] = 0.f;
      const int n_col = (t - s0 + TPR) / TPR;  // how many of this thread's columns lie at or below the diagonal
      for (int d = 0; d < dim; d += 4) {
        float4 q4 = *reinterpret_cast<const float4*>(sQ + t * ld + d);
#pragma unroll
        for (int j = 0; j < CPT; ++j) {
          if (j < n_col) {
            float4 k4 = *reinterpret_cast<const float4*>(sK + (s0 + TPR * j) * ld + d);
            acc[j] = fmaf(q4.x, k4.x, acc[j]); acc[j] = fmaf(q4.y, k4.y, acc[j]);
            acc[j] = fmaf(q4.z, k4.z, acc[j]); acc[j] = fmaf(q4.w, k4.w, acc[j]);
          }
        }
      }
      const float M_t = __shfl_sync(0xffffffffu, M, t);  // every warp holds all tokens' scalars, lane = token
#pragma unroll
      for (int j = 0; j < CPT; ++j) {
        int sidx = s0 + TPR * j;
        float z_s = __shfl_sync(0xffffffffu, z, sidx);
        sP[t * (MLC_L + 1) + sidx] = (sidx <= t && sidx < n_tok) ? acc[j] * expf(z_s - M_t) : 0.f;
      }
    }
    __syncthreads();
    // ---- n_t . q_t = sum_s P[t][s] + carry_t (q_t . n0): a warp takes MLC_ROWS rows, lanes share the sums
    for (int r = 0; r < MLC_ROWS; ++r) {
      const int t = warp * MLC_ROWS + r;
      float part = sP[t * (MLC_L + 1) + lane];
      float qn = 0.f;
      for (int d = lane; d < dim; d += 32) qn = fmaf(sQ[t * ld + d], sn[d], qn);
      part = warp_sum(part);
      qn = warp_sum(qn);
      if (lane == 0) s_nq[t] = part;  // completed below with the row's carry times q_t . n0
      if (lane == 1) sP[t * (MLC_L + 1) + MLC_L] = qn;  // the spare column keeps q_t . n0
    }
    __syncthreads();
    // ---- numerators: thread = (column, MLC_ROWS rows); then the outputs
    {
      const int r0 = warp * MLC_ROWS;
      float acc[MLC_ROWS];
#pragma unroll
      for (int r = 0; r < MLC_ROWS; ++r) acc[r] = 0.f;
      for (int d = 0; d < dim; d += 4) {
        float s0v = sS[d * 32 + lane], s1v = sS[(d + 1) * 32 + lane], s2v = sS[(d + 2) * 32 + lane], s3v = sS[(d + 3) * 32 + lane];
#pragma unroll
        for (int r = 0; r < MLC_ROWS; ++r) {
          float4 q4 = *reinterpret_cast<const float4*>(sQ + (r0 + r) * ld + d);
          acc[r] = fmaf(q4.x, s0v, acc[r]); acc[r] = fmaf(q4.y, s1v, acc[r]);
          acc[r] = fmaf(q4.z, s2v, acc[r]); acc[r] = fmaf(q4.w, s3v, acc[r]);
        }
      }
#pragma unroll
      for (int r = 0; r < MLC_ROWS; ++r) acc[r] *= __shfl_sync(0xffffffffu, carry, r0 + r);
      for (int sidx = 0; sidx < n_tok; ++sidx) {
        float v = sV[sidx * 32 + lane];
#pragma unroll
        for (int r = 0; r < MLC_ROWS; ++r) acc[r] = fmaf(sP[(r0 + r) * (MLC_L + 1) + sidx], v, acc[r]);
      }
#pragma unroll
      for (int r = 0; r < MLC_ROWS; ++r) {
        const int t = r0 + r;
        float nq = s_nq[t] + __shfl_sync(0xffffffffu, carry, t) * sP[t * (MLC_L + 1) + MLC_L];
        float denom = fmaxf(fabsf(nq), expf(-__shfl_sync(0xffffffffu, m_tok, t))) + 1e-6f;
        if (t < n_tok && has_col) out[(size_t)(base + t) * n_heads * vdim + (size_t)head * vdim + c] = acc[r] / denom;
      }
    }
    __syncthreads();  // everyone has read sS and sn as they were before the chunk
    // ---- the state after the chunk: thread = (column, eight rows d at a time; the warps take turns)
    for (int dbase = warp * 8; dbase < dim; dbase += 8 * (MLC_THREADS / 32)) {
      float acc[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] = 0.f;
      for (int sidx = 0; sidx < n_tok; ++sidx) {
        const float gv = s_g[sidx] * sV[sidx * 32 + lane];
#pragma unroll
        for (int j = 0; j < 8; j += 4) {
          // rows are padded by four and followed by other arrays: a read past dim stays inside and is not kept
          float4 k4 = *reinterpret_cast<const float4*>(sK + sidx * ld + dbase + j);
          acc[j] = fmaf(gv, k4.x, acc[j]);         acc[j + 1] = fmaf(gv, k4.y, acc[j + 1]);
          acc[j + 2] = fmaf(gv, k4.z, acc[j + 2]); acc[j + 3] = fmaf(gv, k4.w, acc[j + 3]);
        }
      }
#pragma unroll
      for (int j = 0; j < 8; ++j)
        if (dbase + j < dim) sS[(dbase + j) * 32 + lane] = fmaf(carry_last, sS[(dbase + j) * 32 + lane], acc[j]);
    }
    for (int d = tid; d < dim; d += MLC_THREADS) {
      float acc = 0.f;
      for (int sidx = 0; sidx < n_tok; ++sidx) acc = fmaf(s_g[sidx], sK[sidx * ld + d], acc);
      sn[d] = fmaf(carry_last, sn[d], acc);
    }
    m0 = m_end;
  }
  __syncthreads();
  for (int i = tid; i < dim * 32; i += MLC_THREADS) {
    int d = i >> 5, cc = i & 31;
    if (c0 + cc < vdim) st[(size_t)d * vdim + c0 + cc] = sS[i];
  }
  if (blockIdx.z == 0) {
    for (int d = tid; d < dim; d += MLC_THREADS) st_n[d] = sn[d];
    if (tid == 0) st_n[dim] = m0;
  }
}

// As bn_mlstm_recurrence, by chunks of 32 tokens (for steps that bring runs of many tokens).
extern "C" int bn_mlstm_chunks(const void* qkv, int dtype, int row_stride, int k_off, int v_off, const float* gates,
                               float* state, const int* seq_start, const int* slots, int n_seqs, int n_heads, int dim,
                               int vdim, float q_scale, float* out, cudaStream_t stream) {
  if (n_seqs <= 0) return BN_OK;
  if (!qkv || !gates || !state || !out || n_heads <= 0 || dim <= 0 || dim % 4 || vdim <= 0 || n_heads > 65535 ||
      (vdim + 31) / 32 > 65535)
    return BN_ERR_BAD_ARG;
  size_t floats = 2 * (size_t)MLC_L * (dim + 4) + (size_t)dim * 32 + MLC_L * 32 + MLC_L * (MLC_L + 1) + dim + 2 * MLC_L;
  size_t smem = floats * sizeof(float);
  if (smem > 200 * 1024) return BN_ERR_BAD_ARG;
  dim3 grid(n_seqs, n_heads, (vdim + 31) / 32);
  static size_t granted_f = 0, granted_b = 0;
  if (dtype == BN_F32) {
    if (smem > 48 * 1024 && smem > granted_f) {
      cudaError_t e = cudaFuncSetAttribute(mlstm_chunk_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (e != cudaSuccess) return BN_ERR_LAUNCH + (int)e;
      granted_f = smem;
    }
    BN_LAUNCH(mlstm_chunk_kernel<float>, grid, MLC_THREADS, smem, stream, (const float*)qkv, row_stride, k_off, v_off, gates,
              state, seq_start, slots, n_heads, dim, vdim, q_scale, out);
  } else if (dtype == BN_BF16) {
    if (smem > 48 * 1024 && smem > granted_b) {
      cudaError_t e = cudaFuncSetAttribute(mlstm_chunk_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (e != cudaSuccess) return BN_ERR_LAUNCH + (int)e;
      granted_b = smem;
    }
    BN_LAUNCH(mlstm_chunk_kernel<__nv_bfloat16>, grid, MLC_THREADS, smem, stream, (const __nv_bfloat16*)qkv, row_stride, k_off,
              v_off, gates, state, seq_start, slots, n_heads, dim, vdim, q_scale, out);
  } else {
    return BN_ERR_BAD_ARG;
  }
  BN_CHECK_LAUNCH();
  return BN_OK;
}

// out[t][h][c] = o[t][h][c] / sqrt(mean_c(o[t][h]^2) + eps) * gain[h * vdim + c] * sigmoid(g[t][h * vdim + c])
template <typename T, typename W>
__global__ void mlstm_output_kernel(const float* __restrict__ o, const W* __restrict__ gain, const T* __restrict__ g,
                                    int g_stride, int n_heads, int vdim, float eps, T* __restrict__ out) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = blockDim.x >> 5;
  for (int h = warp; h < n_heads; h += n_warps) {
    const float* oh = o + ((size_t)t * n_heads + h) * vdim;
    float ss = 0.f;
    for (int c = lane; c < vdim; c += 32) ss = fmaf(oh[c], oh[c], ss);
    ss = warp_sum(ss);
    float scale = 1.0f / sqrtf(ss / (float)vdim + eps);
    for (int c = lane; c < vdim; c += 32) {
      float gate = 1.0f / (1.0f + expf(-to_f32<T>(g[(size_t)t * g_stride + (size_t)h * vdim + c])));
      out[((size_t)t * n_heads + h) * vdim + c] = from_f32<T>(oh[c] * scale * to_f32<W>(gain[(size_t)h * vdim + c]) * gate);
    }
  }
}

extern "C" int bn_mlstm_output(const float* o, const void* gain, int gain_dtype, const void* g, int g_stride, int dtype,
                               int n_tokens, int n_heads, int vdim, float eps, void* out, cudaStream_t stream) {
  if (n_tokens <= 0) return BN_OK;
  if (!o || !gain || !g || !out || n_heads <= 0 || vdim <= 0 || !(eps > 0.f)) return BN_ERR_BAD_ARG;
  if (dtype == BN_F32 && gain_dtype == BN_F32)
    BN_LAUNCH((mlstm_output_kernel<float, float>), n_tokens, 128, 0, stream, o, (const float*)gain, (const float*)g,
              g_stride, n_heads, vdim, eps, (float*)out);
  else if (dtype == BN_BF16 && gain_dtype == BN_BF16)
    BN_LAUNCH((mlstm_output_kernel<__nv_bfloat16, __nv_bfloat16>), n_tokens, 128, 0, stream, o, (const __nv_bfloat16*)gain,
              (const __nv_bfloat16*)g, g_stride, n_heads, vdim, eps, (__nv_bfloat16*)out);
  else if (dtype == BN_BF16 && gain_dtype == BN_F32)
    BN_LAUNCH((mlstm_output_kernel<__nv_bfloat16, float>), n_tokens, 128, 0, stream, o, (const float*)gain,
              (const __nv_bfloat16*)g, g_stride, n_heads, vdim, eps, (__nv_bfloat16*)out);
  else
    return BN_ERR_BAD_ARG;
  BN_CHECK_LAUNCH();
  return BN_OK;
}
