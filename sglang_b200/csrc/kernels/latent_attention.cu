// Absorbed latent attention over a paged cache, with a sliding window and per-head soft-max sinks.
//
// The cache holds ONE latent row c_j of R numbers per token; keys and values of all heads are linear maps of it, and those maps are applied
// outside this kernel (query side: q~ = W_uk^T q; output side: W_uv o~).  What runs here is multi-query attention over the latent rows:
//     p_j  = exp(scale * q~ . c_j - m) / (sum_j' exp(scale * q~ . c_j' - m) + exp(sink - m))    for keys 0 <= i - j < window
//     o~   = sum_j p_j c_j
// One kernel serves prompt portions (QT = 8 queries of a request per CTA) and decode (QT = 1).  A CTA owns QT consecutive queries x HG heads
// (HG chosen on the host so that the tile fits shared memory).  It walks the keys its queries can see — the window plus QT - 1 — in tiles of
// 32: the tile's latent rows go to shared memory once (fp32, row stride R + 1) and are used by every (query, head) pair as key AND as value.
// A warp owns whole pairs: lane = key for the scores (R multiply-adds against a broadcast query), lane = latent column for the output
// (probabilities broadcast by shuffle), running max / sum in registers, output accumulator in shared memory.  The sink is the initial
// state of the running soft-max (m = sink, l = 1, o = 0), so it is counted once and needs no branch at the end.  All arithmetic is fp32.
#include "common.cuh"
#include "tma_host.h"

namespace sglb {
namespace {

constexpr int KT = 32;           // keys per tile (= lanes)
constexpr int NW = 8;            // warps per CTA

template <typename T> __device__ __forceinline__ float ldc(const T* p);
template <> __device__ __forceinline__ float ldc<float>(const float* p) { return *p; }
template <> __device__ __forceinline__ float ldc<__nv_bfloat16>(const __nv_bfloat16* p) { return __bfloat162float(*p); }

struct LatentParams {
  const float* q; float* out;                 // [T, H, R]
  const void* cache; int ldc;                 // rows of ldc elements, the first R are the latent
  const int* page_table; int pt_stride; int page_size;
  const int* req_slots; const int* seq_lens; const int* cu_q;
  const float* sinks;
  int H, R, HG, window;
  float scale;
};

template <typename TCache, int QT>
__global__ void __launch_bounds__(NW * 32) latent_attention_kernel(const LatentParams p) {
  extern __shared__ float sm[];
  const int b = blockIdx.y;
  const int qbase = p.cu_q ? p.cu_q[b] : b;
  const int n = p.cu_q ? p.cu_q[b + 1] - qbase : 1;
  const int t0 = blockIdx.x * QT;
  if (t0 >= n) return;
  const int nq = min(QT, n - t0);
  const int L = p.seq_lens[b];
  const int pos0 = L - n + t0;                 // position of the CTA's first query
  const int h0 = blockIdx.z * p.HG;
  const int nh = min(p.HG, p.H - h0);
  const int R = p.R, RP = R + 1;
  const int P = nq * nh;                       // (query, head) pairs of this CTA: pair = qi * nh + hi
  float* s_q = sm;                             // [QT * HG][R]
  float* s_o = s_q + QT * p.HG * R;            // [QT * HG][R]
  float* s_c = s_o + QT * p.HG * R;            // [KT][R + 1]
  int* s_slot = (int*)(s_c + KT * RP);         // [KT]
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  for (int idx = tid; idx < P * R; idx += NW * 32) {
    const int pr = idx / R, r = idx - pr * R;
    const int qi = pr / nh, hi = pr - qi * nh;
    s_q[idx] = p.q[((size_t)(qbase + t0 + qi) * p.H + h0 + hi) * R + r];
    s_o[idx] = 0.f;
  }
  // running soft-max state of the pairs this warp owns (pair = warp + k * NW)
  constexpr int PPW_MAX = 16;
  float m_run[PPW_MAX], l_run[PPW_MAX];
#pragma unroll
  for (int k = 0; k < PPW_MAX; ++k) {
    const int pr = warp + k * NW;
    const float sink = (p.sinks && pr < P) ? p.sinks[h0 + pr % nh] : -INFINITY;
    m_run[k] = sink;
    l_run[k] = p.sinks ? 1.f : 0.f;
  }
  const int last = pos0 + nq - 1;
  const int first = p.window > 0 ? max(0, pos0 - p.window + 1) : 0;
  const int* pt = p.page_table + (size_t)p.req_slots[b] * p.pt_stride;
  const TCache* cache = (const TCache*)p.cache;
  for (int k0 = first; k0 <= last; k0 += KT) {
    __syncthreads();                           // the previous tile is consumed (and s_q / s_o are initialised)
    if (tid < KT) {
      const int kp = k0 + tid;
      s_slot[tid] = kp <= last ? pt[kp / p.page_size] * p.page_size + kp % p.page_size : -1;
    }
    __syncthreads();
    for (int idx = tid; idx < KT * R; idx += NW * 32) {
      const int k = idx / R, r = idx - k * R;
      const int slot = s_slot[k];
      s_c[k * RP + r] = slot >= 0 ? ldc<TCache>(cache + (size_t)slot * p.ldc + r) : 0.f;
    }
    __syncthreads();
    const int kp = k0 + lane;
#pragma unroll
    for (int k = 0; k < PPW_MAX; ++k) {
      const int pr = warp + k * NW;
      if (pr >= P) break;
      const int qi = pr / nh;
      const int qpos = pos0 + qi;
      const int lo = p.window > 0 ? qpos - p.window + 1 : 0;
      if (k0 > qpos || k0 + KT - 1 < lo) continue;          // no key of this tile is visible to the pair (warp-uniform)
      const bool vis = kp <= qpos && kp >= lo;
      const float* qv = s_q + pr * R;
      const float* cv = s_c + lane * RP;
      float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
      int r = 0;
      for (; r + 4 <= R; r += 4) {
        a0 += qv[r] * cv[r];
        a1 += qv[r + 1] * cv[r + 1];
        a2 += qv[r + 2] * cv[r + 2];
        a3 += qv[r + 3] * cv[r + 3];
      }
      for (; r < R; ++r) a0 += qv[r] * cv[r];
      const float s = vis ? ((a0 + a1) + (a2 + a3)) * p.scale : -INFINITY;
      const float m_new = fmaxf(m_run[k], warp_max(s));
      if (m_new == -INFINITY) continue;
      const float alpha = m_run[k] == -INFINITY ? 0.f : expf(m_run[k] - m_new);
      const float pj = vis ? expf(s - m_new) : 0.f;
      l_run[k] = l_run[k] * alpha + warp_sum(pj);
      m_run[k] = m_new;
      float* ov = s_o + pr * R;
      for (int c0 = 0; c0 < R; c0 += 128) {                 // 4 column groups per pass: one shuffle feeds 4 multiply-adds
        float acc[4] = {0.f, 0.f, 0.f, 0.f};
        int cc[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) cc[u] = min(c0 + 32 * u + lane, R - 1);
#pragma unroll 8
        for (int j = 0; j < KT; ++j) {
          const float pb = __shfl_sync(0xffffffffu, pj, j);
#pragma unroll
          for (int u = 0; u < 4; ++u) acc[u] += pb * s_c[j * RP + cc[u]];
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int c = c0 + 32 * u + lane;
          if (c < R) ov[c] = ov[c] * alpha + acc[u];
        }
      }
    }
  }
  __syncwarp();
#pragma unroll
  for (int k = 0; k < PPW_MAX; ++k) {
    const int pr = warp + k * NW;
    if (pr >= P) break;
    const int qi = pr / nh, hi = pr - qi * nh;
    const float inv = 1.f / l_run[k];
    float* dst = p.out + ((size_t)(qbase + t0 + qi) * p.H + h0 + hi) * R;
    for (int c = lane; c < R; c += 32) dst[c] = s_o[pr * R + c] * inv;
  }
}

template <typename TCache, int QT>
void launch(LatentParams p, int B, int max_q_len, cudaStream_t stream) {
  // heads per CTA: as many as fit 200 KB next to the key tile, at most 16 pairs per warp
  const size_t tile = (size_t)KT * (p.R + 1) * 4 + KT * 4;
  const size_t per_head = (size_t)QT * p.R * 4 * 2;
  int hg = (int)std::min<size_t>((size_t)p.H, (200 * 1024 - tile) / per_head);
  hg = std::min(hg, 16 * NW / QT);
  if (hg < 1) throw std::runtime_error("sglb latent_attention: latent rank too large for one CTA");
  p.HG = hg;
  const size_t smem = tile + per_head * hg;
  auto kern = latent_attention_kernel<TCache, QT>;
  if (smem > 48 * 1024) SGLB_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  dim3 grid((max_q_len + QT - 1) / QT, B, (p.H + hg - 1) / hg);
  kern<<<grid, NW * 32, smem, stream>>>(p);
  SGLB_CUDA_CHECK(cudaGetLastError());
}

}  // namespace

void latent_attention(const float* q, const void* cache, bool cache_bf16, int ldc, int R, const int* page_table, int pt_stride, int page_size,
                      const int* req_slots, const int* seq_lens, const int* cu_q, int B, int max_q_len, int H, float scale, int window,
                      const float* sinks, float* out, cudaStream_t stream) {
  if (B <= 0 || max_q_len <= 0) return;
  if (B > 65535) throw std::runtime_error("sglb latent_attention: more than 65535 requests in one call");
  LatentParams p;
  p.q = q; p.out = out; p.cache = cache; p.ldc = ldc; p.page_table = page_table; p.pt_stride = pt_stride; p.page_size = page_size;
  p.req_slots = req_slots; p.seq_lens = seq_lens; p.cu_q = cu_q; p.sinks = sinks; p.H = H; p.R = R; p.HG = 1; p.window = window; p.scale = scale;
  const bool decode = cu_q == nullptr || max_q_len == 1;
  if (cache_bf16) {
    if (decode) launch<__nv_bfloat16, 1>(p, B, 1, stream); else launch<__nv_bfloat16, 8>(p, B, max_q_len, stream);
  } else {
    if (decode) launch<float, 1>(p, B, 1, stream); else launch<float, 8>(p, B, max_q_len, stream);
  }
}

}  // namespace sglb
