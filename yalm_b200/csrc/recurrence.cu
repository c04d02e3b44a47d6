// A gated linear recurrence per head whose forget gate also decides what is written:
//   S_t = diag(f_t) S_(t-1) + (1 - f_t) v_t^T,   o_t = S_t^T q_t,
// S [key size, value size] per head and sequence, carried from step to step in 32-bit floats.
// Everything here is 32-bit.  Two kernels:
//
//  * recurrence_gates: the fused projection [q | f | v] of a step (split-K slices) with its
//    activations applied, q = silu(.), f = l + (1 - l) sigmoid(. + bias) with a lower bound l per
//    key channel, v as it is: one pass over the step's tokens, all in parallel;
//  * recurrence_scan: the recurrence itself.  A block owns RC_COLS value columns of one
//    (sequence, head), a warp RC_CPW of them, and a lane RPT neighbouring rows of those columns'
//    state in registers.  The step's tokens of the sequence come through a three-stage cp.async ring,
//    RC_TOK tokens per stage (one block barrier per stage); a token costs a lane RPT state
//    updates and RPT multiply-adds, and the 32 partial sums of an output are added for RC_TOK
//    tokens at once, so that the shuffles of different tokens overlap.
#include "api.h"
#include "common.cuh"

namespace yalm {

constexpr int RC_CPW = 2;                 // value columns per warp
constexpr int RC_COLS = 8 * RC_CPW;       // ... per block of eight warps
constexpr int RC_TOK = 16;
constexpr int RC_STAGES = 3;

// grid (token, part of the row): a thread takes four elements of the row, a block 1,024, so that
// a decode step's few tokens still spread over many blocks.
__global__ void recurrence_gates_kernel(const float* __restrict__ proj, int n_partials,
                                        long long partial_stride, const float* __restrict__ f_bias,
                                        const float* __restrict__ lower, float* __restrict__ act,
                                        int row, int n_q) {
  pdl_launch_dependents();
  pdl_wait();
  const size_t base = (size_t)blockIdx.x * row;
  const int e_end = min(row, (int)(blockIdx.y + 1) * 1024);
  for (int e = blockIdx.y * 1024 + threadIdx.x; e < e_end; e += blockDim.x) {
    const float z = sum_slices(proj + base + e, n_partials, partial_stride);
    float v = z;
    if (e < n_q) {
      v = z / (1.0f + expf(-z));
    } else if (e < 2 * n_q) {
      const float l = lower[e - n_q];
      v = l + (1.0f - l) * (1.0f / (1.0f + expf(-(z + f_bias[e - n_q]))));
    }
    act[base + e] = v;
  }
}

template <int BYTES>
__device__ __forceinline__ void cp_async(float* dst, const float* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], %2;" ::"r"(smem_u32(dst)), "l"(src), "n"(BYTES) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

// VEC: floats per copy (4 when every offset is a multiple of 16 bytes, else 1)
template <int RPT, int VEC>
__global__ void __launch_bounds__(256)
recurrence_scan_kernel(const float* __restrict__ act, const int* __restrict__ q_start,
                       const int* __restrict__ seq_slot, float* __restrict__ state,
                       float* __restrict__ out, int H, int dk, int dv) {
  pdl_launch_dependents();
  constexpr int DKP = 32 * RPT;                       // rows, padded
  constexpr int PER_TOK = 2 * DKP + RC_COLS;          // q, f, then this block's v columns
  extern __shared__ __align__(16) float stage[];      // [RC_STAGES][RC_TOK][PER_TOK]
  const int b = blockIdx.z, h = blockIdx.y, c0 = blockIdx.x * RC_COLS;
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  const int col = c0 + w * RC_CPW;
  const int slot = seq_slot[b];
  const int t0 = q_start[b], t1 = q_start[b + 1];
  const int row = 2 * H * dk + H * dv;
  // rows beyond dk: f = 0 and q = 0 for ever (never copied over); their state is not stored.
  // Value columns beyond dv are never copied either and nothing of them is stored.
  if (dk < DKP) {
    for (int i = threadIdx.x; i < RC_STAGES * RC_TOK * PER_TOK; i += blockDim.x) stage[i] = 0.f;
    __syncthreads();
  }
  // what this thread copies of every token: up to five runs of VEC floats
  const int per = 2 * dk + RC_COLS;
  int src_off[5], dst_off[5];
#pragma unroll
  for (int k = 0; k < 5; ++k) {
    const int e = (threadIdx.x + k * 256) * VEC;
    src_off[k] = dst_off[k] = -1;
    if (e < dk) { src_off[k] = h * dk + e; dst_off[k] = e; }
    else if (e < 2 * dk) { src_off[k] = H * dk + h * dk + (e - dk); dst_off[k] = DKP + (e - dk); }
    else if (e < per && c0 + (e - 2 * dk) < dv) {
      src_off[k] = 2 * H * dk + h * dv + c0 + (e - 2 * dk);
      dst_off[k] = 2 * DKP + (e - 2 * dk);
    }
  }
  pdl_wait();
  float S[RPT][RC_CPW];
  float* st = state + (((size_t)slot * H + h) * dk) * dv + col;
  // The block's part of the state is dk rows of RC_COLS neighbouring floats.  Where 16-byte
  // accesses fit, it goes through shared memory (a warp reads eight whole 64-byte runs per load)
  // instead of every lane picking its own rows out of memory 8 bytes at a time.
  constexpr int TP = RC_COLS + 1;                     // tile pitch
  const bool tiled = VEC == 4 && c0 + RC_COLS <= dv;
  float* tile_g = state + (((size_t)slot * H + h) * dk) * dv + c0;
  if (tiled) {
    for (int i = threadIdx.x; i < dk * (RC_COLS / 4); i += blockDim.x) {
      const int r = i / (RC_COLS / 4), q4 = i % (RC_COLS / 4);
      const float4 v = *reinterpret_cast<const float4*>(tile_g + (size_t)r * dv + 4 * q4);
      float* d = stage + r * TP + 4 * q4;
      d[0] = v.x; d[1] = v.y; d[2] = v.z; d[3] = v.w;
    }
    __syncthreads();
#pragma unroll
    for (int r = 0; r < RPT; ++r)
#pragma unroll
      for (int c = 0; c < RC_CPW; ++c) {
        const int i = lane * RPT + r;
        S[r][c] = i < dk ? stage[i * TP + w * RC_CPW + c] : 0.f;
      }
    __syncthreads();
    if (dk < DKP) {                                   // the tile lay over rows that must read as zero
      for (int i = threadIdx.x; i < dk * TP; i += blockDim.x) stage[i] = 0.f;
      __syncthreads();
    }
  } else {
#pragma unroll
    for (int r = 0; r < RPT; ++r)
#pragma unroll
      for (int c = 0; c < RC_CPW; ++c) {
        const int i = lane * RPT + r;
        S[r][c] = (col + c < dv && i < dk) ? st[(size_t)i * dv + c] : 0.f;
      }
  }
  const int n_groups = (t1 - t0 + RC_TOK - 1) / RC_TOK;
  auto issue = [&](int g) {
    if (g < n_groups) {
      const int base = t0 + g * RC_TOK;
      const int nt = min(RC_TOK, t1 - base);
      float* dst = stage + (size_t)(g % RC_STAGES) * RC_TOK * PER_TOK;
      const float* src = act + (size_t)base * row;
#pragma unroll
      for (int k = 0; k < 5; ++k)
        if (src_off[k] >= 0)
          for (int tt = 0; tt < nt; ++tt)
            cp_async<4 * VEC>(dst + tt * PER_TOK + dst_off[k], src + (size_t)tt * row + src_off[k]);
    }
    cp_async_commit();
  };
  issue(0);
  issue(1);
  for (int g = 0; g < n_groups; ++g) {
    cp_async_wait<RC_STAGES - 2>();
    __syncthreads();                                   // stage g has landed; stage g - 1 is no longer read
    issue(g + 2);
    const int base = t0 + g * RC_TOK;
    const int nt = min(RC_TOK, t1 - base);
    const float* sg = stage + (size_t)(g % RC_STAGES) * RC_TOK * PER_TOK;
    float o[RC_TOK][RC_CPW];
#pragma unroll
    for (int tt = 0; tt < RC_TOK; ++tt) {
#pragma unroll
      for (int c = 0; c < RC_CPW; ++c) o[tt][c] = 0.f;
      if (tt < nt) {
        const float* q = sg + tt * PER_TOK + lane * RPT;
        const float* f = q + DKP;
        float vj[RC_CPW];
#pragma unroll
        for (int c = 0; c < RC_CPW; ++c) vj[c] = sg[tt * PER_TOK + 2 * DKP + w * RC_CPW + c];
#pragma unroll
        for (int r = 0; r < RPT; ++r) {
          const float fi = f[r], qi = q[r], gi = 1.0f - fi;
#pragma unroll
          for (int c = 0; c < RC_CPW; ++c) {
            S[r][c] = fmaf(fi, S[r][c], gi * vj[c]);
            o[tt][c] = fmaf(S[r][c], qi, o[tt][c]);
          }
        }
      }
    }
    // The group's RC_TOK x RC_CPW = 32 outputs, each the sum of the 32 lanes' partial sums: in every
    // round a lane hands half of its values to its partner and adds the partner's other half to its
    // own, so 16 + 8 + 4 + 2 + 1 exchanges leave lane l with the whole sum of value number l
    // (token l / RC_CPW, column l % RC_CPW).
    static_assert(RC_TOK * RC_CPW == 32, "one output per lane");
    float* ov = &o[0][0];                              // value number tt * RC_CPW + c
#pragma unroll
    for (int half = 16; half >= 1; half >>= 1) {
      const bool upper = (lane & half) != 0;
#pragma unroll
      for (int i = 0; i < half; ++i) {
        const float send = upper ? ov[i] : ov[i + half];
        const float keep = upper ? ov[i + half] : ov[i];
        ov[i] = keep + __shfl_xor_sync(0xffffffffu, send, half);
      }
    }
    {
      const int tt = lane / RC_CPW, c = lane % RC_CPW;
      if (tt < nt && col + c < dv) out[((size_t)(base + tt) * H + h) * dv + col + c] = ov[0];
    }
  }
  cp_async_wait<0>();
  if (tiled) {
    __syncthreads();                                   // the last group's rows are no longer read
#pragma unroll
    for (int r = 0; r < RPT; ++r)
#pragma unroll
      for (int c = 0; c < RC_CPW; ++c) {
        const int i = lane * RPT + r;
        if (i < dk) stage[i * TP + w * RC_CPW + c] = S[r][c];
      }
    __syncthreads();
    for (int i = threadIdx.x; i < dk * (RC_COLS / 4); i += blockDim.x) {
      const int r = i / (RC_COLS / 4), q4 = i % (RC_COLS / 4);
      const float* d = stage + r * TP + 4 * q4;
      *reinterpret_cast<float4*>(tile_g + (size_t)r * dv + 4 * q4) = make_float4(d[0], d[1], d[2], d[3]);
    }
    return;
  }
#pragma unroll
  for (int r = 0; r < RPT; ++r)
#pragma unroll
    for (int c = 0; c < RC_CPW; ++c) {
      const int i = lane * RPT + r;
      if (col + c < dv && i < dk) st[(size_t)i * dv + c] = S[r][c];
    }
}

}  // namespace yalm

using namespace yalm;

// proj: float32 slices [n_partials][tokens][2 H dk + H dv] = (q | f | v); f_bias, lower [H dk];
// act: float32 scratch [tokens][2 H dk + H dv] (the activated projection); state
// [slots][H][dk][dv] float32, read at the step's start and written at its end; out float32
// [tokens][H dv].  dk up to 512.
extern "C" int yalm_gated_recurrence(const float* proj, int n_partials, long long partial_stride,
                                     const float* f_bias, const float* lower, float* act,
                                     const int* q_start, const int* seq_slot, float* state, float* out,
                                     int n_tokens, int n_seqs, int H, int dk, int dv, cudaStream_t stream) {
  if (n_seqs <= 0 || n_tokens <= 0) return 0;
  if (H <= 0 || dk <= 0 || dv <= 0 || dk > 512 || n_seqs > 65535 || H > 65535) return -2;
  const int row = 2 * H * dk + H * dv;
  if ((row + 1023) / 1024 > 65535) return -4;
  launch_pdl(recurrence_gates_kernel, dim3(n_tokens, (row + 1023) / 1024), dim3(256), 0, stream, proj,
             n_partials, partial_stride, f_bias, lower, act, row, H * dk);
  YALM_LAUNCH_CHECK();
  const dim3 grid((dv + RC_COLS - 1) / RC_COLS, H, n_seqs), block(256);
  const int rpt = (dk + 31) / 32;
  // 16-byte copies where every run starts on a 16-byte boundary; a thread copies up to five runs per token
  const bool vec = dk % 4 == 0 && dv % 4 == 0 && (((uintptr_t)act) & 15) == 0;
  if ((2 * dk + RC_COLS + (vec ? 3 : 0)) / (vec ? 4 : 1) > 5 * 256) return -2;
#define YALM_REC(R)                                                                                 \
  do {                                                                                              \
    const size_t smem = (size_t)RC_STAGES * RC_TOK * (2 * 32 * R + RC_COLS) * sizeof(float);        \
    static bool set = false;                                                                        \
    if (!set && smem > 48 * 1024) {                                                                 \
      cudaError_t e = cudaFuncSetAttribute(recurrence_scan_kernel<R, 4>,                            \
                                           cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
      if (e == cudaSuccess)                                                                         \
        e = cudaFuncSetAttribute(recurrence_scan_kernel<R, 1>,                                      \
                                 cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);           \
      if (e != cudaSuccess) return (int)e;                                                          \
      set = true;                                                                                   \
    }                                                                                               \
    if (vec)                                                                                        \
      launch_pdl(recurrence_scan_kernel<R, 4>, grid, block, smem, stream, (const float*)act,        \
                 q_start, seq_slot, state, out, H, dk, dv);                                         \
    else                                                                                            \
      launch_pdl(recurrence_scan_kernel<R, 1>, grid, block, smem, stream, (const float*)act,        \
                 q_start, seq_slot, state, out, H, dk, dv);                                         \
  } while (0)
  if (rpt <= 1) YALM_REC(1);
  else if (rpt <= 2) YALM_REC(2);
  else if (rpt <= 4) YALM_REC(4);
  else if (rpt <= 8) YALM_REC(8);
  else YALM_REC(16);
#undef YALM_REC
  YALM_LAUNCH_CHECK();
  return 0;
}
