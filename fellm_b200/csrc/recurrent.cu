// Recurrent mixers: what runs between their matrix products.
//
//   causal_conv_act    short causal convolution per channel over portions, then SiLU; history in a state slot
//   token_shift_mix    h + (h_prev - h) * mu_s for several mixes s; the previous row in a state slot
//   lowrank_expand     out = f_out(W2 f_in(z) + bias): the second factor of a low-rank projection, float32
//   delta_scan         gated delta rule:  S = g S; u = beta (v - S^T k); S += k u^T; o = S^T q
//   decay_bonus_scan   o = (S + diag(u) k v^T)^T r; S = diag(w) S + k v^T   (per-channel decay, bonus for the current token)
//   head_norm_gate     per head: o / rms(o) * weight * act(gate)
//   branch_combine     x += mean over branches of rms_unit(branch) * weight
//
// FeLLM's GatedDeltaNet keeps the same two things between steps, a convolution history and a matrix
// (crates/fellm-model/src/graph.rs:792-806), and runs one token per request and step; here a request
// brings a portion of any length and its state after the portion equals the state after the same
// tokens one by one: every sum below runs in an order that depends on the sizes alone, not on where
// a prompt was cut, on the batch, or on the slot.
//
// States, decays, gates of the recurrences, unit norms and every sum are float32 in both engine dtypes.
#include "common.cuh"

#define MAX_TAPS 8
#define CH_TILE 32

__device__ __forceinline__ float silu_f(float z) { return z / (1.0f + expf(-z)); }
__device__ __forceinline__ float sigmoid_f(float z) { return 1.0f / (1.0f + expf(-z)); }
__device__ __forceinline__ float softplus_f(float z) { return z > 20.f ? z : log1pf(expf(z)); }

// ---------------------------------------------------------------- short causal convolution + activation
// grid (channel tiles, items), block (CH_TILE, row lanes).  out[t, c] = act(sum_j taps[c, j] in[t - (L-1) + j, c]);
// inputs before the portion come from the slot's history (the last L-1 inputs; zeros for a new request).
template <typename TA>
__global__ void causal_conv_act_kernel(const TA* __restrict__ x, int ldx, const float* __restrict__ taps, int L,
                                       float* __restrict__ state, long long slot_stride,
                                       const int* __restrict__ item_start, const int* __restrict__ item_slot,
                                       TA* __restrict__ out, int ldo, int C, int act) {
  __shared__ float hist[MAX_TAPS - 1][CH_TILE];
  const int item = blockIdx.y, tx = threadIdx.x;
  const int c = blockIdx.x * CH_TILE + tx;
  const int r0 = item_start[item], n = item_start[item + 1] - r0;
  float* st = state + (size_t)item_slot[item] * slot_stride;
  const bool live = c < C;
  if (threadIdx.y == 0 && live)
    for (int j = 0; j < L - 1; ++j) hist[j][tx] = st[(size_t)j * C + c];
  __syncthreads();
  float w[MAX_TAPS];
#pragma unroll
  for (int j = 0; j < MAX_TAPS; ++j) w[j] = (live && j < L) ? taps[(size_t)c * L + j] : 0.f;
  if (live) {
    for (int r = threadIdx.y; r < n; r += blockDim.y) {
      float acc = 0.f;
#pragma unroll
      for (int j = 0; j < MAX_TAPS; ++j) {
        if (j < L) {
          int idx = r - (L - 1) + j;
          float v = idx >= 0 ? to_f(x[(size_t)(r0 + idx) * ldx + c]) : hist[L - 1 + idx][tx];
          acc = fmaf(w[j], v, acc);
        }
      }
      out[(size_t)(r0 + r) * ldo + c] = from_f<TA>(act == 1 ? silu_f(acc) : acc);
    }
  }
  __syncthreads();
  if (threadIdx.y == 0 && live) {
    float keep[MAX_TAPS - 1];
#pragma unroll
    for (int j = 0; j < MAX_TAPS - 1; ++j) {
      if (j < L - 1) {
        int idx = n - (L - 1) + j;
        keep[j] = idx >= 0 ? to_f(x[(size_t)(r0 + idx) * ldx + c]) : hist[L - 1 + idx][tx];
      }
    }
#pragma unroll
    for (int j = 0; j < MAX_TAPS - 1; ++j)
      if (j < L - 1) st[(size_t)j * C + c] = keep[j];
  }
}

FELLM_API int fellm_causal_conv_act(const void* x, int is_bf16, int ldx, const float* taps, int L, float* state,
                                    long long slot_stride, const int* item_start, const int* item_slot, void* out,
                                    int ldo, int n_items, int C, int act, int all_single, cudaStream_t stream) {
  if (n_items <= 0 || C <= 0) return 0;
  if (L < 1 || L > MAX_TAPS) return FELLM_ERR_SIZE;
  if (!x || !taps || (!state && L > 1) || !item_start || !item_slot || !out) return FELLM_ERR_ARG;
  dim3 grid(ceil_div(C, CH_TILE), n_items), block(CH_TILE, all_single ? 1 : 8);
  if (is_bf16)
    causal_conv_act_kernel<bf16><<<grid, block, 0, stream>>>((const bf16*)x, ldx, taps, L, state, slot_stride, item_start,
                                                             item_slot, (bf16*)out, ldo, C, act);
  else
    causal_conv_act_kernel<float><<<grid, block, 0, stream>>>((const float*)x, ldx, taps, L, state, slot_stride, item_start,
                                                              item_slot, (float*)out, ldo, C, act);
  return launch_status();
}

// ---------------------------------------------------------------- token shift
// out[s][t][c] = h[t][c] + (h[t-1][c] - h[t][c]) * mu[s][c]; the row before a portion is the slot's state, which
// then takes the portion's last row.  Same grid as the convolution.
template <typename TA>
__global__ void token_shift_mix_kernel(const TA* __restrict__ h, const float* __restrict__ mu, int n_mix,
                                       float* __restrict__ state, long long slot_stride,
                                       const int* __restrict__ item_start, const int* __restrict__ item_slot,
                                       TA* __restrict__ out, int T, int d) {
  const int item = blockIdx.y;
  const int c = blockIdx.x * CH_TILE + threadIdx.x;
  if (c >= d) return;
  const int r0 = item_start[item], n = item_start[item + 1] - r0;
  float* st = state + (size_t)item_slot[item] * slot_stride;
  const float first_prev = threadIdx.y == 0 ? st[c] : 0.f;     // row 0 belongs to row lane 0, which is also the one writer below
  for (int r = threadIdx.y; r < n; r += blockDim.y) {
    float cur = to_f(h[(size_t)(r0 + r) * d + c]);
    float prev = r > 0 ? to_f(h[(size_t)(r0 + r - 1) * d + c]) : first_prev;
    float diff = prev - cur;
    for (int s = 0; s < n_mix; ++s)
      out[((size_t)s * T + r0 + r) * d + c] = from_f<TA>(fmaf(diff, mu[(size_t)s * d + c], cur));
  }
  if (threadIdx.y == 0 && n > 0) st[c] = to_f(h[(size_t)(r0 + n - 1) * d + c]);
}

FELLM_API int fellm_token_shift_mix(const void* h, int is_bf16, const float* mu, int n_mix, float* state,
                                    long long slot_stride, const int* item_start, const int* item_slot, void* out,
                                    int T, int n_items, int d, int all_single, cudaStream_t stream) {
  if (n_items <= 0 || d <= 0) return 0;
  if (!h || !mu || !state || !item_start || !item_slot || !out || n_mix < 1) return FELLM_ERR_ARG;
  dim3 grid(ceil_div(d, CH_TILE), n_items), block(CH_TILE, all_single ? 1 : 8);
  if (is_bf16)
    token_shift_mix_kernel<bf16><<<grid, block, 0, stream>>>((const bf16*)h, mu, n_mix, state, slot_stride, item_start,
                                                             item_slot, (bf16*)out, T, d);
  else
    token_shift_mix_kernel<float><<<grid, block, 0, stream>>>((const float*)h, mu, n_mix, state, slot_stride, item_start,
                                                              item_slot, (float*)out, T, d);
  return launch_status();
}

// ---------------------------------------------------------------- second factor of a low-rank projection
// out[t, n] = f_out(bias[n] + sum_r W2[n, r] f_in(z[t, r])), float32.  f_in: 0 identity, 1 tanh.
// f_out: 0 identity; 1 exp(-exp(v)) (a decay from its double logarithm); 2 exp(-exp(rate[n / per]) softplus(v)).
#define LR_ROWS 8
template <typename TW>
__global__ void __launch_bounds__(128)
lowrank_expand_kernel(const float* __restrict__ z, int ldz, const TW* __restrict__ W2, const float* __restrict__ bias,
                      const float* __restrict__ rate, int per, float* __restrict__ out, int T, int N, int R,
                      int f_in, int f_out) {
  extern __shared__ float zs[];                      // [LR_ROWS][R]
  const int t0 = blockIdx.y * LR_ROWS;
  for (int e = threadIdx.x; e < LR_ROWS * R; e += blockDim.x) {
    int i = e / R, r = e - i * R;
    float v = t0 + i < T ? z[(size_t)(t0 + i) * ldz + r] : 0.f;
    zs[e] = f_in == 1 ? tanhf(v) : v;
  }
  __syncthreads();
  const int n = blockIdx.x * blockDim.x + threadIdx.x;
  if (n >= N) return;
  float acc[LR_ROWS];
#pragma unroll
  for (int i = 0; i < LR_ROWS; ++i) acc[i] = 0.f;
  const TW* wr = W2 + (size_t)n * R;
  for (int r = 0; r < R; ++r) {
    float w = to_f(wr[r]);
#pragma unroll
    for (int i = 0; i < LR_ROWS; ++i) acc[i] = fmaf(zs[i * R + r], w, acc[i]);
  }
  const float b = bias ? bias[n] : 0.f;
  const float rt = f_out == 2 ? expf(rate[n / per]) : 0.f;
#pragma unroll
  for (int i = 0; i < LR_ROWS; ++i) {
    if (t0 + i >= T) break;
    float v = acc[i] + b;
    if (f_out == 1) v = expf(-expf(v));
    else if (f_out == 2) v = expf(-rt * softplus_f(v));
    out[(size_t)(t0 + i) * N + n] = v;
  }
}

FELLM_API int fellm_lowrank_expand(const float* z, int ldz, const void* W2, int w_bf16, const float* bias,
                                   const float* rate, int per, float* out, int T, int N, int R, int f_in, int f_out,
                                   cudaStream_t stream) {
  if (T <= 0 || N <= 0) return 0;
  if (!z || !W2 || !out || R < 1 || (f_out == 2 && (!rate || per < 1))) return FELLM_ERR_ARG;
  if (R > 1024) return FELLM_ERR_SIZE;
  dim3 grid(ceil_div(N, 128), ceil_div(T, LR_ROWS));
  size_t smem = (size_t)LR_ROWS * R * sizeof(float);
  if (w_bf16)
    lowrank_expand_kernel<bf16><<<grid, 128, smem, stream>>>(z, ldz, (const bf16*)W2, bias, rate, per, out, T, N, R, f_in, f_out);
  else
    lowrank_expand_kernel<float><<<grid, 128, smem, stream>>>(z, ldz, (const float*)W2, bias, rate, per, out, T, N, R, f_in, f_out);
  return launch_status();
}

// ---------------------------------------------------------------- the two scans
// A warp owns CPW = 32 / KS columns of one head's matrix S [dk, dv]; a column's dk rows are spread over KS lanes
// (row i = ks + KS * r, r < RMAX), so that a thread keeps at most RMAX values.  Columns are independent of one
// another in both recurrences; sums over dk run over r in a thread, then over the KS lanes by a butterfly.
#define RMAX 32

__device__ __forceinline__ float group_sum(float v, int ks_lanes) {
  for (int o = 1; o < ks_lanes; o <<= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// Gated delta rule.  qkv [T, ldq]: q heads at column 0 (G x dk), k at k_off, v at v_off (H x dv), after their
// convolutions and SiLU.  small [T, lds]: beta's logit at column b_off + h; per-head decay: logit at a_off + h,
// g = exp(-exp(A_log[h]) softplus(logit + dt_bias[h])); per-channel decay: gch [T, H*dk] holds g itself.
template <typename TA>
__global__ void __launch_bounds__(128)
delta_scan_kernel(const TA* __restrict__ qkv, int ldq, int k_off, int v_off, const float* __restrict__ small, int lds,
                  int b_off, int a_off, const float* __restrict__ A_log, const float* __restrict__ dt_bias,
                  const float* __restrict__ gch, float* __restrict__ state, long long slot_stride,
                  const int* __restrict__ item_start, const int* __restrict__ item_slot, float* __restrict__ out,
                  int H, int G, int dk, int dv, int KS, int col_groups) {
  const int warp = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  const int item = blockIdx.y;
  if (warp >= H * col_groups) return;
  const int h = warp / col_groups, cg = warp - h * col_groups;
  const int CPW = 32 / KS, ks = lane % KS;
  const int j = cg * CPW + lane / KS;
  const bool col_live = j < dv;
  const int jc = col_live ? j : dv - 1;
  const int g = h / (H / G);
  const int r0 = item_start[item], n = item_start[item + 1] - r0;
  float* Sg = state + (size_t)item_slot[item] * slot_stride + (size_t)h * dk * dv;
  float S[RMAX];
#pragma unroll
  for (int r = 0; r < RMAX; ++r) {
    int i = ks + KS * r;
    S[r] = i < dk ? Sg[(size_t)i * dv + jc] : 0.f;
  }
  const float rate = gch ? 0.f : expf(A_log[h]);
  const float bias_a = gch ? 0.f : dt_bias[h];
  const float q_scale = 1.0f / sqrtf((float)dk);
  for (int t = 0; t < n; ++t) {
    const size_t row = (size_t)(r0 + t);
    const TA* qr = qkv + row * ldq + (size_t)g * dk;
    const TA* kr = qr + k_off;
    float q[RMAX], k[RMAX];
    float sq = 0.f, sk = 0.f;
#pragma unroll
    for (int r = 0; r < RMAX; ++r) {
      int i = ks + KS * r;
      q[r] = i < dk ? to_f(qr[i]) : 0.f;
      k[r] = i < dk ? to_f(kr[i]) : 0.f;
      sq = fmaf(q[r], q[r], sq);
      sk = fmaf(k[r], k[r], sk);
    }
    sq = group_sum(sq, KS);
    sk = group_sum(sk, KS);
    const float qn = q_scale / sqrtf(sq + 1e-6f), kn = 1.0f / sqrtf(sk + 1e-6f);
    const float v = to_f(qkv[row * ldq + v_off + (size_t)h * dv + jc]);
    const float beta = sigmoid_f(small[row * lds + b_off + h]);
    float dot = 0.f;
    if (gch) {
      const float* gr = gch + row * ((size_t)H * dk) + (size_t)h * dk;
#pragma unroll
      for (int r = 0; r < RMAX; ++r) {
        int i = ks + KS * r;
        k[r] *= kn;
        S[r] *= i < dk ? gr[i] : 0.f;
        dot = fmaf(S[r], k[r], dot);
      }
    } else {
      const float gt = expf(-rate * softplus_f(small[row * lds + a_off + h] + bias_a));
#pragma unroll
      for (int r = 0; r < RMAX; ++r) {
        k[r] *= kn;
        S[r] *= gt;
        dot = fmaf(S[r], k[r], dot);
      }
    }
    dot = group_sum(dot, KS);
    const float u = beta * (v - dot);
    float o = 0.f;
#pragma unroll
    for (int r = 0; r < RMAX; ++r) {
      S[r] = fmaf(k[r], u, S[r]);
      o = fmaf(S[r], q[r], o);
    }
    o = group_sum(o, KS) * qn;
    if (ks == 0 && col_live) out[row * ((size_t)H * dv) + (size_t)h * dv + j] = o;
  }
  if (col_live) {
#pragma unroll
    for (int r = 0; r < RMAX; ++r) {
      int i = ks + KS * r;
      if (i < dk) Sg[(size_t)i * dv + j] = S[r];
    }
  }
}

static int scan_lanes(int dk) {
  int ks = 1;
  while (ks * RMAX < dk) ks <<= 1;
  return ks;
}

FELLM_API int fellm_delta_scan(const void* qkv, int is_bf16, int ldq, int k_off, int v_off, const float* small, int lds,
                               int b_off, int a_off, const float* A_log, const float* dt_bias, const float* gch,
                               float* state, long long slot_stride, const int* item_start, const int* item_slot,
                               float* out, int n_items, int H, int G, int dk, int dv, cudaStream_t stream) {
  if (n_items <= 0) return 0;
  if (dk < 1 || dk > 32 * RMAX || dv < 1 || G < 1 || H % G) return FELLM_ERR_SIZE;
  if (!qkv || !small || !state || !item_start || !item_slot || !out || (!gch && (!A_log || !dt_bias))) return FELLM_ERR_ARG;
  const int KS = scan_lanes(dk), CPW = 32 / KS;
  const int col_groups = ceil_div(dv, CPW);
  const int warps = H * col_groups;
  dim3 grid(ceil_div(warps, 4), n_items);
  if (is_bf16)
    delta_scan_kernel<bf16><<<grid, 128, 0, stream>>>((const bf16*)qkv, ldq, k_off, v_off, small, lds, b_off, a_off, A_log,
                                                      dt_bias, gch, state, slot_stride, item_start, item_slot, out, H, G, dk,
                                                      dv, KS, col_groups);
  else
    delta_scan_kernel<float><<<grid, 128, 0, stream>>>((const float*)qkv, ldq, k_off, v_off, small, lds, b_off, a_off, A_log,
                                                       dt_bias, gch, state, slot_stride, item_start, item_slot, out, H, G, dk,
                                                       dv, KS, col_groups);
  return launch_status();
}

// Decay-and-bonus recurrence.  r, k, v [T, ld] (H x dk each), w float32 [T, H*dk] (the decay itself), u [H, dk].
template <typename TA>
__global__ void __launch_bounds__(128)
decay_bonus_scan_kernel(const TA* __restrict__ rr, const TA* __restrict__ kk, const TA* __restrict__ vv, int ld,
                        const float* __restrict__ w, const float* __restrict__ u, float* __restrict__ state,
                        long long slot_stride, const int* __restrict__ item_start, const int* __restrict__ item_slot,
                        float* __restrict__ out, int H, int dk, int KS, int col_groups) {
  const int warp = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  const int item = blockIdx.y;
  if (warp >= H * col_groups) return;
  const int h = warp / col_groups, cg = warp - h * col_groups;
  const int CPW = 32 / KS, ks = lane % KS;
  const int j = cg * CPW + lane / KS;
  const bool col_live = j < dk;
  const int jc = col_live ? j : dk - 1;
  const int r0 = item_start[item], n = item_start[item + 1] - r0;
  float* Sg = state + (size_t)item_slot[item] * slot_stride + (size_t)h * dk * dk;
  float S[RMAX], bonus[RMAX];
#pragma unroll
  for (int r = 0; r < RMAX; ++r) {
    int i = ks + KS * r;
    S[r] = i < dk ? Sg[(size_t)i * dk + jc] : 0.f;
    bonus[r] = i < dk ? u[(size_t)h * dk + i] : 0.f;
  }
  for (int t = 0; t < n; ++t) {
    const size_t row = (size_t)(r0 + t);
    const size_t base = row * ld + (size_t)h * dk;
    const float* wr = w + row * ((size_t)H * dk) + (size_t)h * dk;
    const float vj = to_f(vv[base + jc]);
    float o = 0.f;
#pragma unroll
    for (int r = 0; r < RMAX; ++r) {
      int i = ks + KS * r;
      if (i < dk) {
        float kv = to_f(kk[base + i]) * vj;
        o = fmaf(to_f(rr[base + i]), fmaf(bonus[r], kv, S[r]), o);
        S[r] = fmaf(wr[i], S[r], kv);
      }
    }
    o = group_sum(o, KS);
    if (ks == 0 && col_live) out[row * ((size_t)H * dk) + (size_t)h * dk + j] = o;
  }
  if (col_live) {
#pragma unroll
    for (int r = 0; r < RMAX; ++r) {
      int i = ks + KS * r;
      if (i < dk) Sg[(size_t)i * dk + j] = S[r];
    }
  }
}

FELLM_API int fellm_decay_bonus_scan(const void* r, const void* k, const void* v, int is_bf16, int ld, const float* w,
                                     const float* u, float* state, long long slot_stride, const int* item_start,
                                     const int* item_slot, float* out, int n_items, int H, int dk, cudaStream_t stream) {
  if (n_items <= 0) return 0;
  if (dk < 1 || dk > 32 * RMAX || H < 1) return FELLM_ERR_SIZE;
  if (!r || !k || !v || !w || !u || !state || !item_start || !item_slot || !out) return FELLM_ERR_ARG;
  const int KS = scan_lanes(dk), CPW = 32 / KS;
  const int col_groups = ceil_div(dk, CPW);
  dim3 grid(ceil_div(H * col_groups, 4), n_items);
  if (is_bf16)
    decay_bonus_scan_kernel<bf16><<<grid, 128, 0, stream>>>((const bf16*)r, (const bf16*)k, (const bf16*)v, ld, w, u, state,
                                                            slot_stride, item_start, item_slot, out, H, dk, KS, col_groups);
  else
    decay_bonus_scan_kernel<float><<<grid, 128, 0, stream>>>((const float*)r, (const float*)k, (const float*)v, ld, w, u,
                                                             state, slot_stride, item_start, item_slot, out, H, dk, KS,
                                                             col_groups);
  return launch_status();
}

// ---------------------------------------------------------------- per-head norm and gate
// y[t, h, e] = o[t, h, e] / sqrt(mean_e o^2 + eps) * w[(per_head ? h * dv : 0) + e] * act(gate[t, h*dv + e]);
// act: 0 no gate, 1 SiLU, 2 sigmoid.  One warp per (t, h).
template <typename TO, typename TG>
__global__ void __launch_bounds__(128)
head_norm_gate_kernel(const float* __restrict__ o, const float* __restrict__ w, int per_head,
                      const TG* __restrict__ gate, int ldg, int act, TO* __restrict__ y, int T, int H, int dv, float eps) {
  const int warp = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (warp >= T * H) return;
  const int t = warp / H, h = warp - t * H;
  const float* orow = o + ((size_t)t * H + h) * dv;
  float ss = 0.f;
  for (int e = lane; e < dv; e += 32) { float v = orow[e]; ss = fmaf(v, v, ss); }
  ss = warp_sum(ss);
  const float scale = 1.0f / sqrtf(ss / (float)dv + eps);
  const float* wr = w + (per_head ? (size_t)h * dv : 0);
  TO* yr = y + ((size_t)t * H + h) * dv;
  for (int e = lane; e < dv; e += 32) {
    float v = (orow[e] * scale) * wr[e];
    if (act) {
      float gz = to_f(gate[(size_t)t * ldg + (size_t)h * dv + e]);
      v *= act == 1 ? silu_f(gz) : sigmoid_f(gz);
    }
    yr[e] = from_f<TO>(v);
  }
}

FELLM_API int fellm_head_norm_gate(const float* o, const float* w, int per_head, const void* gate, int gate_bf16, int ldg,
                                   int act, void* y, int y_bf16, int T, int H, int dv, float eps, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (!o || !w || !y || (act && !gate)) return FELLM_ERR_ARG;
  unsigned blocks = (unsigned)(((long long)T * H + 3) / 4);
#define HNG(TO_, TG_) head_norm_gate_kernel<TO_, TG_><<<blocks, 128, 0, stream>>>(o, w, per_head, (const TG_*)gate, ldg, act, (TO_*)y, T, H, dv, eps)
  if (y_bf16) { if (gate_bf16) HNG(bf16, bf16); else HNG(bf16, float); }
  else { if (gate_bf16) HNG(float, bf16); else HNG(float, float); }
#undef HNG
  return launch_status();
}

// ---------------------------------------------------------------- branches of a parallel mixer
// x[t, :] += (1 / n) * sum_b branch_b[t, :] / sqrt(mean(branch_b[t]^2) + eps) * w_b.  One block per row.
#define MAX_BRANCHES 4
struct Branches { const float* o[MAX_BRANCHES]; const float* w[MAX_BRANCHES]; };

__global__ void __launch_bounds__(256)
branch_combine_kernel(Branches br, int n_br, float* __restrict__ x, int d, float eps) {
  __shared__ float part[MAX_BRANCHES][8];
  __shared__ float scale[MAX_BRANCHES];
  const int t = blockIdx.x;
  for (int b = 0; b < n_br; ++b) {
    const float* o = br.o[b] + (size_t)t * d;
    float ss = 0.f;
    for (int e = threadIdx.x; e < d; e += blockDim.x) ss = fmaf(o[e], o[e], ss);
    ss = warp_sum(ss);
    if ((threadIdx.x & 31) == 0) part[b][threadIdx.x >> 5] = ss;
  }
  __syncthreads();
  if (threadIdx.x < n_br) {
    float s = 0.f;
    for (int i = 0; i < (int)(blockDim.x >> 5); ++i) s += part[threadIdx.x][i];
    scale[threadIdx.x] = 1.0f / sqrtf(s / (float)d + eps);
  }
  __syncthreads();
  const float inv = 1.0f / (float)n_br;
  for (int e = threadIdx.x; e < d; e += blockDim.x) {
    float s = 0.f;
    for (int b = 0; b < n_br; ++b) s += (br.o[b][(size_t)t * d + e] * scale[b]) * br.w[b][e];
    x[(size_t)t * d + e] += s * inv;
  }
}

FELLM_API int fellm_branch_combine(const float* const* outs, const float* const* weights, int n_br, float* x, int T, int d,
                                   float eps, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (n_br < 1 || n_br > MAX_BRANCHES) return FELLM_ERR_SIZE;
  if (!outs || !weights || !x) return FELLM_ERR_ARG;
  Branches br;
  for (int b = 0; b < MAX_BRANCHES; ++b) { br.o[b] = b < n_br ? outs[b] : nullptr; br.w[b] = b < n_br ? weights[b] : nullptr; }
  branch_combine_kernel<<<T, 256, 0, stream>>>(br, n_br, x, d, eps);
  return launch_status();
}
