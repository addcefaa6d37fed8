// Gated delta rule over a ragged batch: prompt portions and single decode tokens run the same kernel.
//
// Per (request, value head) the fp32 matrix state S [Dk, Dv] follows, token by token,
//     S <- g * S                    g: one decay per head, or one per head and key channel (acts on the rows of S)
//     w  = beta * (v - S^T k)
//     S <- S + k w^T
//     o  = S^T q                    (after the write)
// with q, k the unit vectors of the short-convolution outputs (q also / sqrt(Dk)), beta = sigmoid(b_raw),
// g = exp(-exp(A_log) * softplus(a_raw + dt_bias)); the read-out is RMS-normalised per head, weighted and gated (silu | sigmoid).
//
// Mapping: one CTA per (value head, request).  The columns of S are independent in every step, so a column lives in the registers of KS
// neighbouring lanes (ROWS rows each, interleaved: row = r * KS + ks); S^T k and S^T q are per-lane dot products closed by log2(KS)
// shuffles.  Tokens are staged TC at a time: all warps normalise q / k, evaluate decay and beta and copy v into shared memory, the
// recurrence runs TC steps out of shared memory (broadcast reads), then the warps normalise and gate the TC outputs.  Only the chunk
// boundaries need CTA barriers.  The state is read once and written once per call; a request whose cached length is zero starts from
// S = 0 whatever its slot holds.  Everything is fp32.
//
// The order of operations per token does not depend on how a prompt was cut or batched, so a position's output is bit-identical across
// schedules.  A long single prompt is a serial chain of T steps per head; a chunk-parallel (WY / UT transform) tensor-core kernel is the
// known next step for that regime.
#include "common.cuh"
#include "tma_host.h"

namespace sglb {
namespace {

constexpr int TC = 8;            // tokens staged per chunk

struct DeltaParams {
  const float* u; int ldu; int k_off; int v_off;        // conv outputs [T, ldu]: q at 0, k at k_off, v at v_off
  const float* a_raw; int a_ld;                          // [T, a_ld]: a_ld = H (per head) or H * Dk (per channel)
  const float* b_raw;                                    // [T, H]
  const float* gate_raw;                                 // [T, H * Dv] or null
  const float* A_log; const float* dt_bias; const float* norm_w;
  float* state;                                          // [slots, H, Dk, Dv]
  const int* req_slots; const int* seq_lens; const int* cu_q;
  float* out;                                            // [T, H, Dv]
  int H, rep, Dk, Dv, per_channel, gate_silu;
  float eps, q_scale;
};

__device__ __forceinline__ float softplus_f(float x) { return x > 20.f ? x : log1pf(expf(x)); }

template <int ROWS, int KS, int MAXT>
__global__ void __launch_bounds__(MAXT) gated_delta_rule_kernel(const DeltaParams p) {
  extern __shared__ float sm[];
  const int h = blockIdx.x, b = blockIdx.y;
  const int q0 = p.cu_q ? p.cu_q[b] : b;
  const int n = p.cu_q ? p.cu_q[b + 1] - q0 : 1;
  if (n <= 0) return;
  const int Dk = p.Dk, Dv = p.Dv, H = p.H;
  const int hk = h / p.rep;
  float* s_q = sm;                           // [TC][Dk]
  float* s_k = s_q + TC * Dk;                // [TC][Dk]
  float* s_g = s_k + TC * Dk;                // [TC][Dk] (per channel) or [TC]
  float* s_v = s_g + (p.per_channel ? TC * Dk : TC);   // [TC][Dv]
  float* s_o = s_v + TC * Dv;                // [TC][Dv]
  float* s_beta = s_o + TC * Dv;             // [TC]
  const int tid = threadIdx.x, nthr = blockDim.x, warp = tid >> 5, lane = tid & 31, nwarp = nthr >> 5;
  const int col = tid / KS, ks = tid % KS;
  const bool live = col < Dv;
  float S[ROWS];
  float* st = p.state + ((size_t)p.req_slots[b] * H + h) * Dk * Dv;
  const bool fresh = p.seq_lens[b] - n == 0;
#pragma unroll
  for (int r = 0; r < ROWS; ++r) {
    const int i = r * KS + ks;
    S[r] = (live && !fresh && i < Dk) ? st[(size_t)i * Dv + col] : 0.f;
  }
  const float a_exp = expf(p.A_log[h]);
  for (int t0 = 0; t0 < n; t0 += TC) {
    const int tc = min(TC, n - t0);
    // ---- stage: one warp per token normalises q and k, evaluates decay and beta; all threads copy v
    for (int tt = warp; tt < tc; tt += nwarp) {
      const float* row = p.u + (size_t)(q0 + t0 + tt) * p.ldu;
      float sq = 0.f, sk = 0.f;
      for (int i = lane; i < Dk; i += 32) {
        const float qv = row[hk * Dk + i], kv = row[p.k_off + hk * Dk + i];
        sq += qv * qv;
        sk += kv * kv;
      }
      sq = warp_sum(sq);
      sk = warp_sum(sk);
      const float rq = p.q_scale / sqrtf(sq + 1e-6f), rk = 1.f / sqrtf(sk + 1e-6f);
      for (int i = lane; i < Dk; i += 32) {
        s_q[tt * Dk + i] = row[hk * Dk + i] * rq;
        s_k[tt * Dk + i] = row[p.k_off + hk * Dk + i] * rk;
      }
      const float* ar = p.a_raw + (size_t)(q0 + t0 + tt) * p.a_ld;
      if (p.per_channel) {
        for (int i = lane; i < Dk; i += 32) s_g[tt * Dk + i] = expf(-a_exp * softplus_f(ar[h * Dk + i] + p.dt_bias[h * Dk + i]));
      } else if (lane == 0) {
        s_g[tt] = expf(-a_exp * softplus_f(ar[h] + p.dt_bias[h]));
      }
      if (lane == 0) s_beta[tt] = 1.f / (1.f + expf(-p.b_raw[(size_t)(q0 + t0 + tt) * H + h]));
    }
    for (int idx = tid; idx < tc * Dv; idx += nthr) {
      const int tt = idx / Dv, j = idx - tt * Dv;
      s_v[idx] = p.u[(size_t)(q0 + t0 + tt) * p.ldu + p.v_off + h * Dv + j];
    }
    __syncthreads();
    // ---- recurrence
    for (int tt = 0; tt < tc; ++tt) {
      const float* kq = s_k + tt * Dk;
      float acc0 = 0.f, acc1 = 0.f;
      if (p.per_channel) {
        const float* gg = s_g + tt * Dk;
#pragma unroll
        for (int r = 0; r < ROWS; ++r) {
          const int i = r * KS + ks;
          if (i < Dk) {
            S[r] *= gg[i];
            if (r & 1) acc1 += S[r] * kq[i]; else acc0 += S[r] * kq[i];
          }
        }
      } else {
        const float g = s_g[tt];
#pragma unroll
        for (int r = 0; r < ROWS; ++r) {
          const int i = r * KS + ks;
          if (i < Dk) {
            S[r] *= g;
            if (r & 1) acc1 += S[r] * kq[i]; else acc0 += S[r] * kq[i];
          }
        }
      }
      float acc = acc0 + acc1;
#pragma unroll
      for (int o = 1; o < KS; o <<= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
      const float w = s_beta[tt] * ((live ? s_v[tt * Dv + col] : 0.f) - acc);
      const float* qq = s_q + tt * Dk;
      float o0 = 0.f, o1 = 0.f;
#pragma unroll
      for (int r = 0; r < ROWS; ++r) {
        const int i = r * KS + ks;
        if (i < Dk) {
          S[r] += kq[i] * w;
          if (r & 1) o1 += S[r] * qq[i]; else o0 += S[r] * qq[i];
        }
      }
      float o = o0 + o1;
#pragma unroll
      for (int s = 1; s < KS; s <<= 1) o += __shfl_xor_sync(0xffffffffu, o, s);
      if (live && ks == 0) s_o[tt * Dv + col] = o;
    }
    __syncthreads();
    // ---- read-out: per-head RMS norm, weight, gate
    for (int tt = warp; tt < tc; tt += nwarp) {
      float* dst = p.out + ((size_t)(q0 + t0 + tt) * H + h) * Dv;
      if (p.norm_w) {
        float ss = 0.f;
        for (int j = lane; j < Dv; j += 32) ss += s_o[tt * Dv + j] * s_o[tt * Dv + j];
        ss = warp_sum(ss);
        const float rs = 1.f / sqrtf(ss / (float)Dv + p.eps);
        const float* gr = p.gate_raw + (size_t)(q0 + t0 + tt) * H * Dv + (size_t)h * Dv;
        for (int j = lane; j < Dv; j += 32) {
          const float z = gr[j];
          const float sg = 1.f / (1.f + expf(-z));
          dst[j] = s_o[tt * Dv + j] * rs * p.norm_w[j] * (p.gate_silu ? z * sg : sg);
        }
      } else {
        for (int j = lane; j < Dv; j += 32) dst[j] = s_o[tt * Dv + j];
      }
    }
    __syncthreads();
  }
  if (live) {
#pragma unroll
    for (int r = 0; r < ROWS; ++r) {
      const int i = r * KS + ks;
      if (i < Dk) st[(size_t)i * Dv + col] = S[r];
    }
  }
}

template <int ROWS, int KS, int MAXT>
void launch(const DeltaParams& p, int B, cudaStream_t stream) {
  const int threads = ((p.Dv * KS + 31) / 32) * 32;
  const size_t smem = sizeof(float) * ((size_t)TC * p.Dk * 2 + (p.per_channel ? (size_t)TC * p.Dk : TC) + (size_t)TC * p.Dv * 2 + TC);
  auto kern = gated_delta_rule_kernel<ROWS, KS, MAXT>;
  if (smem > 48 * 1024) SGLB_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  kern<<<dim3(p.H, B), threads, smem, stream>>>(p);
  SGLB_CUDA_CHECK(cudaGetLastError());
}

}  // namespace

// returns false when the shape is outside what one CTA per head can hold (see the dispatch at the end)
bool gated_delta_rule(const float* u, int ldu, int Hk, int Dk, int H, int Dv, const float* a_raw, bool per_channel, const float* A_log,
                      const float* dt_bias, const float* b_raw, const float* gate_raw, const float* norm_w, float eps, bool gate_silu, float* state,
                      const int* req_slots, const int* seq_lens, const int* cu_q, int B, float* out, cudaStream_t stream) {
  if (B <= 0) return true;
  if (B > 65535) return false;
  DeltaParams p;
  p.u = u; p.ldu = ldu; p.k_off = Hk * Dk; p.v_off = 2 * Hk * Dk;
  p.a_raw = a_raw; p.a_ld = per_channel ? H * Dk : H; p.b_raw = b_raw; p.gate_raw = gate_raw;
  p.A_log = A_log; p.dt_bias = dt_bias; p.norm_w = norm_w; p.state = state;
  p.req_slots = req_slots; p.seq_lens = seq_lens; p.cu_q = cu_q; p.out = out;
  p.H = H; p.rep = H / Hk; p.Dk = Dk; p.Dv = Dv; p.per_channel = per_channel ? 1 : 0; p.gate_silu = gate_silu ? 1 : 0;
  p.eps = eps; p.q_scale = 1.0f / sqrtf((float)Dk);
  // A column of S is split over KS lanes holding ROWS rows each.  32 rows per lane (<= 512 threads, 128 registers) is the default;
  // 16 rows per lane lets a wide value head use up to 1024 threads; 64 rows per lane covers long keys.
  auto slices = [&](int rows) { int ks = 1; while (ks * rows < Dk && ks < 16) ks <<= 1; return ks; };
  int ks = slices(32);
  if (ks * 32 >= Dk && Dv * ks <= 512) {
    switch (ks) {
      case 1: launch<32, 1, 512>(p, B, stream); return true;
      case 2: launch<32, 2, 512>(p, B, stream); return true;
      case 4: launch<32, 4, 512>(p, B, stream); return true;
      case 8: launch<32, 8, 512>(p, B, stream); return true;
      default: launch<32, 16, 512>(p, B, stream); return true;
    }
  }
  ks = slices(16);
  if (ks * 16 >= Dk && Dv * ks <= 1024) {
    switch (ks) {
      case 1: launch<16, 1, 1024>(p, B, stream); return true;
      case 2: launch<16, 2, 1024>(p, B, stream); return true;
      case 4: launch<16, 4, 1024>(p, B, stream); return true;
      case 8: launch<16, 8, 1024>(p, B, stream); return true;
      default: launch<16, 16, 1024>(p, B, stream); return true;
    }
  }
  ks = slices(64);
  if (ks * 64 >= Dk && Dv * ks <= 512) {
    switch (ks) {
      case 1: launch<64, 1, 512>(p, B, stream); return true;
      case 2: launch<64, 2, 512>(p, B, stream); return true;
      case 4: launch<64, 4, 512>(p, B, stream); return true;
      case 8: launch<64, 8, 512>(p, B, stream); return true;
      default: launch<64, 16, 512>(p, B, stream); return true;
    }
  }
  return false;
}

}  // namespace sglb
