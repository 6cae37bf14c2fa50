// Causal GQA attention over the paged cache on CUDA cores, float32 arithmetic: the engine's
// 32-bit attention, and the yardstick of the tensor-core kernels.
//
// FeLLM counterpart: attention_paged_batch_heads, one thread per (row, head) with a serial
// online softmax over the row's length (plugins/cuda_kernels/src/oxide_kernels.rs:4271-4360;
// formulas crates/fellm-plugin-abi/src/attention_provider.rs:175-237): s_j = (q.k_j)*scale,
// m' = max(m, s), l = l*exp(m-m') + sum exp(s-m'), acc = acc*exp(m-m') + sum p_j v_j, out = acc/l.
//
// One warp per (row, head).  Keys are taken in tiles of 32 that start at the first visible
// position (0, position-window+1, or the start of the query's block of `chunk` positions), so the
// order of every sum depends on the query's position alone: not on the cut of the prompt, the
// batch, or the pages.
//
// Beyond FeLLM's attention the kernel takes: values of another size than keys (vd; a page-layer record is
// K [G][tokens][hd] followed by V [G][tokens][vd]), queries read in place from a wider row (ldq), a soft cap on
// the scores (cap * tanh(s / cap)), blocks of `chunk` positions that a query does not look out of, and a gate
// per (row, head) whose sigmoid scales the head's output; a bias by distance, slope[h] * (query position - key
// position) taken off the scaled score; a query temperature by position, q times
// 1 + coef * ln(floor((p + 1) / every) + 1); and values that ARE the keys (vd == 0 in the record: a page-layer
// record then holds the keys alone and the read-out has the keys' size).  kv_write puts a step's keys and values,
// as the product left them, into their pages.
#include "common.cuh"

#define MAX_HD 256

template <typename TA, typename TC>
__global__ void __launch_bounds__(128)
paged_attention_simt_kernel(const TA* __restrict__ q, const TC* __restrict__ pool,
                            const int* __restrict__ block_table, int max_pages,
                            const int* __restrict__ positions, const int* __restrict__ row_slot,
                            TA* __restrict__ out, int T, int H, int G, int hd, int page_tokens, int layer,
                            int layers_in_group, float scale, int window, int vd, int ldq, float softcap, int chunk,
                            const float* __restrict__ gate, int ldg, const float* __restrict__ slopes,
                            float qt_coef, int qt_every) {
  FELLM_TRACE_SCOPE(TRACE_ATTENTION_SIMT);
  extern __shared__ float qs_all[];                 // [warps per block][hd]
  int wib = threadIdx.x >> 5, lane = threadIdx.x & 31;
  int warp = blockIdx.x * (blockDim.x >> 5) + wib;
  if (warp >= T * H) return;
  int row = warp / H, h = warp - row * H;
  int g = h / (H / G);
  float* qs = qs_all + (size_t)wib * hd;
  const TA* qr = q + (size_t)row * ldq + (size_t)h * hd;
  int pos = positions[row];
  const float qt = qt_every > 0 ? 1.0f + qt_coef * logf((float)((pos + 1) / qt_every + 1)) : 1.0f;
  for (int e = lane; e < hd; e += 32) qs[e] = to_f(qr[e]) * qt;
  __syncwarp();
  const float slope = slopes ? slopes[h] : 0.f;
  const bool v_is_k = vd == 0;          // the values are the keys: nothing else is stored
  if (v_is_k) vd = hd;
  const int* bt = block_table + (size_t)row_slot[row] * max_pages;
  int k_begin = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
  if (chunk > 0) k_begin = max(k_begin, (pos / chunk) * chunk);
  const size_t record = (size_t)G * page_tokens * (v_is_k ? hd : hd + vd);       // one page of one layer: keys, then values

  float m = -INFINITY, l = 0.f;
  float acc[MAX_HD / 32];
#pragma unroll
  for (int i = 0; i < MAX_HD / 32; ++i) acc[i] = 0.f;

  for (int k0 = k_begin; k0 <= pos; k0 += 32) {
    int kj = k0 + lane;
    float s = -INFINITY;
    const TC* vrow = nullptr;
    if (kj <= pos) {
      int page = max(bt[kj / page_tokens], 0);      // an unmapped entry (-1) must never become an address
      const TC* rec = pool + ((size_t)page * layers_in_group + layer) * record;
      size_t tok = (size_t)g * page_tokens + (kj % page_tokens);
      const TC* krow = rec + tok * hd;
      vrow = v_is_k ? krow : rec + (size_t)G * page_tokens * hd + tok * vd;
      float dot = 0.f;
      for (int e = 0; e < hd; ++e) dot = fmaf(qs[e], to_f(krow[e]), dot);
      s = dot * scale;
      if (softcap > 0.f) s = softcap * tanhf(s / softcap);
      s -= slope * (float)(pos - kj);
    }
    float m_new = fmaxf(m, warp_max(s));
    float p = kj <= pos ? expf(s - m_new) : 0.f;
    float corr = expf(m - m_new);                  // m = -inf on the first tile: exp(-inf) = 0
    l = l * corr + warp_sum(p);
    m = m_new;
#pragma unroll
    for (int i = 0; i < MAX_HD / 32; ++i) acc[i] *= corr;
    int n_valid = pos - k0 + 1 < 32 ? pos - k0 + 1 : 32;
    for (int j = 0; j < n_valid; ++j) {
      float pj = __shfl_sync(0xffffffffu, p, j);
      const TC* vj = (const TC*)__shfl_sync(0xffffffffu, (unsigned long long)vrow, j);
#pragma unroll
      for (int i = 0; i < MAX_HD / 32; ++i) {
        int e = lane + 32 * i;
        if (e < vd) acc[i] = fmaf(pj, to_f(vj[e]), acc[i]);
      }
    }
  }
  TA* o = out + ((size_t)row * H + h) * vd;
  float inv_l = 1.0f / l;
  if (gate) inv_l *= 1.0f / (1.0f + expf(-gate[(size_t)row * ldg + h]));
#pragma unroll
  for (int i = 0; i < MAX_HD / 32; ++i) {
    int e = lane + 32 * i;
    if (e < vd) o[e] = from_f<TA>(acc[i] * inv_l);
  }
}

// Keys and values of a step's rows into their pages: k at column k_off of a row of `src` (G x hd), v at v_off
// (G x vd).  A row whose page is not mapped writes nothing and sets the status word to 2.
template <typename TA, typename TC>
__global__ void kv_write_kernel(const TA* __restrict__ src, int ld, int k_off, int v_off, TC* __restrict__ pool,
                                const int* __restrict__ block_table, int max_pages, const int* __restrict__ positions,
                                const int* __restrict__ row_slot, int G, int hd, int vd, int page_tokens, int layer,
                                int layers_in_group, int* __restrict__ status) {
  const int row = blockIdx.x;
  const int pos = positions[row];
  const int page = block_table[(size_t)row_slot[row] * max_pages + pos / page_tokens];
  if (page < 0) {
    if (threadIdx.x == 0 && status) atomicExch(status, 2);
    return;
  }
  const size_t record = (size_t)G * page_tokens * (hd + vd);
  TC* rec = pool + ((size_t)page * layers_in_group + layer) * record;
  const int in_page = pos % page_tokens;
  const TA* s = src + (size_t)row * ld;
  for (int e = threadIdx.x; e < G * hd; e += blockDim.x) {
    int g = e / hd, c = e - g * hd;
    rec[((size_t)g * page_tokens + in_page) * hd + c] = from_f<TC>(to_f(s[k_off + e]));
  }
  TC* vrec = rec + (size_t)G * page_tokens * hd;
  for (int e = threadIdx.x; e < G * vd; e += blockDim.x) {
    int g = e / vd, c = e - g * vd;
    vrec[((size_t)g * page_tokens + in_page) * vd + c] = from_f<TC>(to_f(s[v_off + e]));
  }
}

FELLM_API int fellm_kv_write(const void* src, int act_bf16, int ld, int k_off, int v_off, void* pool, int cache_bf16,
                             const int* block_table, int max_pages, const int* positions, const int* row_slot, int T,
                             int G, int hd, int vd, int page_tokens, int layer, int layers_in_group, int* status,
                             cudaStream_t stream) {
  if (T <= 0) return 0;
  if (!src || !pool || !block_table || !positions || !row_slot) return FELLM_ERR_ARG;
  if (act_bf16 != cache_bf16) return FELLM_ERR_ARG;
  if (act_bf16)
    kv_write_kernel<bf16, bf16><<<T, 128, 0, stream>>>((const bf16*)src, ld, k_off, v_off, (bf16*)pool, block_table, max_pages,
                                                       positions, row_slot, G, hd, vd, page_tokens, layer, layers_in_group, status);
  else
    kv_write_kernel<float, float><<<T, 128, 0, stream>>>((const float*)src, ld, k_off, v_off, (float*)pool, block_table,
                                                         max_pages, positions, row_slot, G, hd, vd, page_tokens, layer,
                                                         layers_in_group, status);
  return launch_status();
}

FELLM_API int fellm_paged_attention_general(const void* q, int act_bf16, const void* pool, int cache_bf16,
                                            const int* block_table, int max_pages, const int* positions,
                                            const int* row_slot, void* out, int T, int H, int G, int hd,
                                            int page_tokens, int layer, int layers_in_group, float scale,
                                            int window, int vd, int ldq, float softcap, int chunk, const float* gate,
                                            int ldg, const float* slopes, float qt_coef, int qt_every,
                                            cudaStream_t stream) {
  if (T <= 0) return 0;
  if (hd < 1 || hd > MAX_HD || vd < 0 || vd > MAX_HD) return FELLM_ERR_SIZE;
  if (G < 1 || H % G) return FELLM_ERR_SIZE;
  if (!q || !pool || !block_table || !positions || !row_slot || !out) return FELLM_ERR_ARG;
  if (act_bf16 != cache_bf16) return FELLM_ERR_ARG;
  int warps_per_block = 4;
  long long warps = (long long)T * H;
  unsigned blocks = (unsigned)((warps + warps_per_block - 1) / warps_per_block);
  size_t smem = (size_t)warps_per_block * hd * sizeof(float);
  if (act_bf16)
    paged_attention_simt_kernel<bf16, bf16><<<blocks, warps_per_block * 32, smem, stream>>>((const bf16*)q,
        (const bf16*)pool, block_table, max_pages, positions, row_slot, (bf16*)out, T, H, G, hd, page_tokens,
        layer, layers_in_group, scale, window, vd, ldq, softcap, chunk, gate, ldg, slopes, qt_coef, qt_every);
  else
    paged_attention_simt_kernel<float, float><<<blocks, warps_per_block * 32, smem, stream>>>((const float*)q,
        (const float*)pool, block_table, max_pages, positions, row_slot, (float*)out, T, H, G, hd, page_tokens,
        layer, layers_in_group, scale, window, vd, ldq, softcap, chunk, gate, ldg, slopes, qt_coef, qt_every);
  return launch_status();
}

FELLM_API int fellm_paged_attention_simt(const void* q, int act_bf16, const void* pool, int cache_bf16,
                                         const int* block_table, int max_pages, const int* positions,
                                         const int* row_slot, void* out, int T, int H, int G, int hd,
                                         int page_tokens, int layer, int layers_in_group, float scale,
                                         int window, cudaStream_t stream) {
  return fellm_paged_attention_general(q, act_bf16, pool, cache_bf16, block_table, max_pages, positions, row_slot, out,
                                       T, H, G, hd, page_tokens, layer, layers_in_group, scale, window, hd, H * hd, 0.f,
                                       0, nullptr, 0, nullptr, 0.f, 0, stream);
}
