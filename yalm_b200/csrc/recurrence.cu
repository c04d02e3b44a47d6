// A gated linear recurrence per head whose forget gate also decides what is written:
//   S_t = diag(f_t) S_(t-1) + (1 - f_t) v_t^T,   o_t = S_t^T q_t,
// S [key size, value size] per head and sequence, carried from step to step in 32-bit floats.
// The kernel takes the fused projection [q | f | v] of a step as split-K slices and applies
// the activations itself: q = silu(.), f = l + (1 - l) sigmoid(. + bias) with a lower bound l
// per key channel.  Everything here is 32-bit.
//
// A block owns RC_COLS value columns of one (sequence, head).  Its threads are RC_COLS x
// RC_KS: thread (j, s) keeps the state rows s, s + RC_KS, ... of column j in registers.  The
// step's tokens of the sequence are staged RC_TOK at a time in shared memory (activations
// applied on the way), then walked through without a block barrier; the RC_KS partial sums
// of an output are added inside the warp.
#include "api.h"
#include "common.cuh"

namespace yalm {

constexpr int RC_COLS = 32;
constexpr int RC_KS = 8;
constexpr int RC_TOK = 16;

template <int RPT>
__global__ void __launch_bounds__(RC_COLS * RC_KS)
gated_recurrence_kernel(const float* __restrict__ proj, int n_partials, long long partial_stride,
                        const float* __restrict__ f_bias, const float* __restrict__ lower,
                        const int* __restrict__ q_start, const int* __restrict__ seq_slot,
                        float* __restrict__ state, float* __restrict__ out, int H, int dk, int dv) {
  pdl_launch_dependents();
  extern __shared__ float stage[];                    // [RC_TOK][2 dk + RC_COLS]: q, f, v of a token
  const int b = blockIdx.z, h = blockIdx.y, c0 = blockIdx.x * RC_COLS;
  const int s = threadIdx.x % RC_KS, j = threadIdx.x / RC_KS;
  const int col = c0 + j;
  const bool col_on = col < dv;
  const int slot = seq_slot[b];
  const int t0 = q_start[b], t1 = q_start[b + 1];
  const int row = 2 * H * dk + H * dv;
  const int per_tok = 2 * dk + RC_COLS;
  pdl_wait();
  float S[RPT];
  float* st = state + (((size_t)slot * H + h) * dk) * dv + col;
#pragma unroll
  for (int r = 0; r < RPT; ++r) {
    const int i = s + r * RC_KS;
    S[r] = (col_on && i < dk) ? st[(size_t)i * dv] : 0.f;
  }
  for (int base = t0; base < t1; base += RC_TOK) {
    const int nt = min(RC_TOK, t1 - base);
    __syncthreads();
    for (int idx = threadIdx.x; idx < nt * per_tok; idx += blockDim.x) {
      const int tt = idx / per_tok, e = idx % per_tok;
      const float* src = proj + (size_t)(base + tt) * row;
      float v;
      if (e < dk) {                                    // q = silu(z)
        const float z = sum_slices(src + h * dk + e, n_partials, partial_stride);
        v = z / (1.0f + expf(-z));
      } else if (e < 2 * dk) {                         // f = l + (1 - l) sigmoid(z + bias)
        const int c = h * dk + (e - dk);
        const float z = sum_slices(src + H * dk + c, n_partials, partial_stride) + f_bias[c];
        const float l = lower[c];
        v = l + (1.0f - l) * (1.0f / (1.0f + expf(-z)));
      } else {                                         // v
        const int c = c0 + (e - 2 * dk);
        v = c < dv ? sum_slices(src + 2 * H * dk + h * dv + c, n_partials, partial_stride) : 0.f;
      }
      stage[idx] = v;
    }
    __syncthreads();
    for (int tt = 0; tt < nt; ++tt) {
      const float* q = stage + tt * per_tok;
      const float* f = q + dk;
      const float vj = q[2 * dk + j];
      float o = 0.f;
#pragma unroll
      for (int r = 0; r < RPT; ++r) {
        const int i = s + r * RC_KS;
        if (i < dk) {
          const float fi = f[i];
          S[r] = fmaf(fi, S[r], (1.0f - fi) * vj);
          o = fmaf(S[r], q[i], o);
        }
      }
#pragma unroll
      for (int off = RC_KS / 2; off > 0; off >>= 1) o += __shfl_xor_sync(0xffffffffu, o, off);
      if (s == 0 && col_on) out[((size_t)(base + tt) * H + h) * dv + col] = o;
    }
  }
#pragma unroll
  for (int r = 0; r < RPT; ++r) {
    const int i = s + r * RC_KS;
    if (col_on && i < dk) st[(size_t)i * dv] = S[r];
  }
}

}  // namespace yalm

using namespace yalm;

// proj: float32 slices [n_partials][tokens][2 H dk + H dv] = (q | f | v); f_bias, lower [H dk];
// state [slots][H][dk][dv] float32, read at the step's start and written at its end;
// out float32 [tokens][H dv].  dk up to 256.
extern "C" int yalm_gated_recurrence(const float* proj, int n_partials, long long partial_stride,
                                     const float* f_bias, const float* lower, const int* q_start,
                                     const int* seq_slot, float* state, float* out, int n_seqs, int H,
                                     int dk, int dv, cudaStream_t stream) {
  if (n_seqs <= 0) return 0;
  if (H <= 0 || dk <= 0 || dv <= 0 || dk > 256 || n_seqs > 65535 || H > 65535) return -2;
  const dim3 grid((dv + RC_COLS - 1) / RC_COLS, H, n_seqs), block(RC_COLS * RC_KS);
  const size_t smem = (size_t)RC_TOK * (2 * dk + RC_COLS) * sizeof(float);
  const int rpt = (dk + RC_KS - 1) / RC_KS;
#define YALM_REC(R)                                                                                  \
  launch_pdl(gated_recurrence_kernel<R>, grid, block, smem, stream, proj, n_partials, partial_stride, \
             f_bias, lower, q_start, seq_slot, state, out, H, dk, dv)
  if (rpt <= 2) YALM_REC(2);
  else if (rpt <= 4) YALM_REC(4);
  else if (rpt <= 8) YALM_REC(8);
  else if (rpt <= 16) YALM_REC(16);
  else YALM_REC(32);
#undef YALM_REC
  YALM_LAUNCH_CHECK();
  return 0;
}
