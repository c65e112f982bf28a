// leopard_b200 — minGRU: a gated recurrence whose gates read only the current token, so a prompt is a parallel scan.
//
//   z_t = sigmoid(a_t + bz), u_t = b_t + bx, candidate c_t = u_t + 1/2 (u_t >= 0) | sigmoid(u_t) (u_t < 0)
//   S_t = (1 - z_t) S_(t-1) + z_t c_t   per channel, S_(-1) = 0;   out_t = S_t * silu(g_t)
// a, b, g are the three column blocks of one fp32 projection; gates, candidate and state are fp32.  State [slot][width].
//
//   prompts   chunks of LP_RETENTION_CHUNK tokens (the batch's chunk tables): (1) per chunk and channel the pair (A, B) with
//             S_end = A S_start + B, in parallel; (2) per request and channel a scan over its chunks that leaves every chunk's start
//             state in the workspace, from the stored state when the request has history; (3) per chunk and channel the recurrence
//             again from the start state, writing the gated outputs; the request's last chunk stores the final state.
//   decode    one thread per (request, channel).
#include "lp_host.h"
#include "../../include/leopard_b200.h"

namespace lp {

typedef __nv_bfloat16 bf16;

struct GruArgs {
  const float* zxg; long long ld; int z_off, x_off, g_off;
  int width;
  const float* z_bias; const float* x_bias;
  float* state; long long slot_stride;
  void* out; long long ldo; int out_fp32;
};

__device__ __forceinline__ float gru_sigmoid(float v) { return 1.0f / (1.0f + expf(-v)); }
// one token of one channel: S <- (1 - z) S + z c
__device__ __forceinline__ float gru_step(float S, float a_pre, float b_pre) {
  const float z = gru_sigmoid(a_pre);
  const float c = b_pre >= 0.f ? b_pre + 0.5f : gru_sigmoid(b_pre);
  return fmaf(z, c, (1.0f - z) * S);
}
__device__ __forceinline__ void gru_store(const GruArgs& a, long long row, int ch, float S) {
  const float g = a.zxg[row * a.ld + a.g_off + ch];
  const float v = S * (g / (1.0f + expf(-g)));
  if (a.out_fp32) reinterpret_cast<float*>(a.out)[row * a.ldo + ch] = v;
  else reinterpret_cast<bf16*>(a.out)[row * a.ldo + ch] = __float2bfloat16(v);
}

constexpr int GRU_THREADS = 128;

__global__ void __launch_bounds__(GRU_THREADS)
mingru_chunk_kernel(GruArgs a, const int* __restrict__ chunk_row0, const int* __restrict__ chunk_len, float* __restrict__ ws, int n_chunks) {
  const int c = blockIdx.x, ch = blockIdx.y * GRU_THREADS + threadIdx.x;
  if (ch >= a.width) return;
  const int row0 = chunk_row0[c], len = chunk_len[c];
  const float bz = a.z_bias != nullptr ? a.z_bias[ch] : 0.f, bx = a.x_bias != nullptr ? a.x_bias[ch] : 0.f;
  float A = 1.f, B = 0.f;
  for (int j = 0; j < len; ++j) {
    const float* x = a.zxg + (long long)(row0 + j) * a.ld;
    const float z = gru_sigmoid(x[a.z_off + ch] + bz);
    const float u = x[a.x_off + ch] + bx;
    const float cand = u >= 0.f ? u + 0.5f : gru_sigmoid(u);
    A *= 1.0f - z;
    B = fmaf(z, cand, (1.0f - z) * B);
  }
  ws[(long long)c * a.width + ch] = A;
  ws[((long long)n_chunks + c) * a.width + ch] = B;
}

__global__ void __launch_bounds__(GRU_THREADS)
mingru_scan_kernel(GruArgs a, const int* __restrict__ seq_chunk0, const int* __restrict__ seq_pos0, const int* __restrict__ seq_slot,
                   float* __restrict__ ws, int n_chunks) {
  const int s = blockIdx.x, ch = blockIdx.y * GRU_THREADS + threadIdx.x;
  if (ch >= a.width) return;
  float S = seq_pos0[s] == 0 ? 0.f : a.state[(long long)seq_slot[s] * a.slot_stride + ch];
  for (int c = seq_chunk0[s]; c < seq_chunk0[s + 1]; ++c) {
    const float A = ws[(long long)c * a.width + ch], B = ws[((long long)n_chunks + c) * a.width + ch];
    ws[(long long)c * a.width + ch] = S;      // the chunk's start state replaces its A
    S = fmaf(A, S, B);
  }
}

__global__ void __launch_bounds__(GRU_THREADS)
mingru_out_kernel(GruArgs a, const int* __restrict__ chunk_seq, const int* __restrict__ chunk_row0, const int* __restrict__ chunk_len,
                  const int* __restrict__ seq_chunk0, const int* __restrict__ seq_slot, const float* __restrict__ ws) {
  const int c = blockIdx.x, ch = blockIdx.y * GRU_THREADS + threadIdx.x;
  if (ch >= a.width) return;
  const int row0 = chunk_row0[c], len = chunk_len[c], s = chunk_seq[c];
  const float bz = a.z_bias != nullptr ? a.z_bias[ch] : 0.f, bx = a.x_bias != nullptr ? a.x_bias[ch] : 0.f;
  float S = ws[(long long)c * a.width + ch];
  for (int j = 0; j < len; ++j) {
    const float* x = a.zxg + (long long)(row0 + j) * a.ld;
    S = gru_step(S, x[a.z_off + ch] + bz, x[a.x_off + ch] + bx);
    gru_store(a, row0 + j, ch, S);
  }
  if (c == seq_chunk0[s + 1] - 1) a.state[(long long)seq_slot[s] * a.slot_stride + ch] = S;
}

__global__ void __launch_bounds__(GRU_THREADS)
mingru_decode_kernel(GruArgs a, const int* __restrict__ seq_row0, const int* __restrict__ seq_pos0, const int* __restrict__ seq_slot) {
  const int s = blockIdx.x, ch = blockIdx.y * GRU_THREADS + threadIdx.x;
  if (ch >= a.width) return;
  const long long row = seq_row0[s];
  float* st = a.state + (long long)seq_slot[s] * a.slot_stride + ch;
  const float bz = a.z_bias != nullptr ? a.z_bias[ch] : 0.f, bx = a.x_bias != nullptr ? a.x_bias[ch] : 0.f;
  const float* x = a.zxg + row * a.ld;
  const float S = gru_step(seq_pos0[s] == 0 ? 0.f : *st, x[a.z_off + ch] + bz, x[a.x_off + ch] + bx);
  *st = S;
  gru_store(a, row, ch, S);
}

static int fill_gru(GruArgs& a, const lp_mingru_desc* d) {
  LP_REQUIRE(d != nullptr && d->zxg != nullptr && d->state != nullptr && d->out != nullptr, "lp_mingru: null operand");
  LP_REQUIRE(d->width > 0, "lp_mingru: bad width %d", d->width);
  a.zxg = d->zxg; a.ld = d->ld; a.z_off = d->z_off; a.x_off = d->x_off; a.g_off = d->g_off;
  a.width = d->width;
  a.z_bias = d->z_bias; a.x_bias = d->x_bias;
  a.state = d->state; a.slot_stride = d->slot_stride;
  a.out = d->out; a.ldo = d->ldo; a.out_fp32 = d->out_fp32;
  return 0;
}

}  // namespace lp

using namespace lp;

extern "C" size_t lp_mingru_workspace_bytes(int n_chunks, int width) { return (size_t)2 * n_chunks * width * sizeof(float); }

extern "C" int lp_mingru_prefill(const lp_mingru_desc* d, int n_seqs, int n_chunks, const int* seq_row0, const int* seq_pos0,
                                 const int* seq_slot, const int* seq_chunk0, const int* chunk_seq, const int* chunk_row0,
                                 const int* chunk_len, void* ws, size_t ws_bytes, void* stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  GruArgs a;
  if (int rc = fill_gru(a, d)) return rc;
  LP_REQUIRE(n_seqs >= 0 && n_chunks >= 0, "lp_mingru_prefill: bad counts");
  if (n_seqs == 0 || n_chunks == 0) return 0;
  LP_REQUIRE(seq_row0 != nullptr && seq_pos0 != nullptr && seq_slot != nullptr && seq_chunk0 != nullptr && chunk_seq != nullptr &&
                 chunk_row0 != nullptr && chunk_len != nullptr, "lp_mingru_prefill: null table");
  LP_REQUIRE(ws != nullptr && ws_bytes >= lp_mingru_workspace_bytes(n_chunks, d->width), "lp_mingru_prefill: workspace too small");
  float* w = reinterpret_cast<float*>(ws);
  const int cy = (d->width + GRU_THREADS - 1) / GRU_THREADS;
  mingru_chunk_kernel<<<dim3(n_chunks, cy), GRU_THREADS, 0, stream>>>(a, chunk_row0, chunk_len, w, n_chunks);
  LP_CHECK_CUDA(cudaGetLastError());
  mingru_scan_kernel<<<dim3(n_seqs, cy), GRU_THREADS, 0, stream>>>(a, seq_chunk0, seq_pos0, seq_slot, w, n_chunks);
  LP_CHECK_CUDA(cudaGetLastError());
  mingru_out_kernel<<<dim3(n_chunks, cy), GRU_THREADS, 0, stream>>>(a, chunk_seq, chunk_row0, chunk_len, seq_chunk0, seq_slot, w);
  LP_CHECK_CUDA(cudaGetLastError());
  note_launch(3);
  return 0;
}

extern "C" int lp_mingru_decode(const lp_mingru_desc* d, int n_seqs, const int* seq_row0, const int* seq_pos0, const int* seq_slot,
                                void* stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  GruArgs a;
  if (int rc = fill_gru(a, d)) return rc;
  LP_REQUIRE(seq_row0 != nullptr && seq_pos0 != nullptr && seq_slot != nullptr, "lp_mingru_decode: null table");
  if (n_seqs <= 0) return 0;
  mingru_decode_kernel<<<dim3(n_seqs, (d->width + GRU_THREADS - 1) / GRU_THREADS), GRU_THREADS, 0, stream>>>(a, seq_row0, seq_pos0, seq_slot);
  note_launch();
  LP_CHECK_CUDA(cudaGetLastError());
  return 0;
}
