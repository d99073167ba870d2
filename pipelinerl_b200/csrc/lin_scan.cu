// Linear recurrences with a matrix state per head, over ragged rows:
//
//     S_t = diag(a_t) S_(t-1) + k_t v_t^T          S: [dk, dv]  (fp32, carried per sequence slot)
//     o_t = S_t^T q_t  (+ skip * v_t)
//
// Two front ends feed the same recurrence:
//   GATED  gated linear attention: q, k, v are columns of the projection buffer, q is scaled, and the decay is a
//          vector per key channel, a = sigmoid(z + bias)^(1/tau), formed as exp(logsigmoid(z + bias) / tau);
//   SSD    state-space duality (Mamba-2): v = x (convolved), k = dt * B, q = C, the decay is one scalar per head,
//          a = exp(-exp(A_log) * dt) with dt = softplus(dt_raw + dt_bias), and skip = D.
// Everything that enters the recurrence is fp32.
//
// Work split: grid (value tiles of 32 columns, heads, segments), 256 threads per CTA.  Thread t owns value column
// t / 8 of the tile and the key channels d = t % 8, t % 8 + 8, ... (R of them, in registers); the 8 partial dot
// products of a column are summed with three shuffles.  A CTA walks its segment token by token (kChunk tokens staged
// in shared memory at a time), so prefill of a chunk and a single decoded token are the same code: a decode step is a
// segment of length 1 whose cost is the state's round trip through HBM.  The state is stored in the order the threads
// hold it, [slot][head][tile][r][thread], so that round trip is fully coalesced; its layout is private to this file.
// The result for a token depends only on the tokens before it in its own sequence: chunk borders, batch composition
// and slot numbers cannot change a bit of it.
#include "prl_common.cuh"

namespace prl {
namespace {

constexpr int kChunk = 8;      // tokens staged per round
constexpr int kColsPerCta = 32;
constexpr int kKeyLanes = 8;

struct ScanArgs {
  // ragged segments
  const int32_t* seg_start; const int32_t* seg_len; const int32_t* seg_slot;
  // recurrence shape
  int heads, dk, dv;
  float* state; int64_t state_slot_stride;      // floats per slot
  float* out; int64_t ld_out;                   // [n, heads*dv] fp32
  // GATED front end
  const float* P; int64_t ldp; int off_q, off_k, off_v; float q_scale;
  const float* z; int64_t ldz; const float* z_bias; float inv_tau;
  // SSD front end
  const float* xbc; int64_t ld_xbc; int groups; int off_dt;
  const float* dt_bias; const float* a_log; const float* skip;
};

__device__ __forceinline__ float softplus_f(float x) { return fmaxf(x, 0.f) + log1pf(expf(-fabsf(x))); }
__device__ __forceinline__ float logsigmoid_f(float x) { return fminf(x, 0.f) - log1pf(expf(-fabsf(x))); }

template <int R, bool SSD>
__global__ void __launch_bounds__(256) lin_scan_kernel(ScanArgs a) {
  extern __shared__ float sm[];
  const int seg = blockIdx.z, h = blockIdx.y, vt = blockIdx.x;
  const int len = a.seg_len[seg];
  if (len <= 0) return;
  const int tid = threadIdx.x, dg = tid % kKeyLanes, vl = tid / kKeyLanes;
  const int v = vt * kColsPerCta + vl;
  const bool v_ok = v < a.dv;
  const int dk = a.dk;
  float* s_a = sm;                       // [kChunk][dk] decay
  float* s_k = s_a + kChunk * dk;        // [kChunk][dk] key coefficient
  float* s_q = s_k + kChunk * dk;        // [kChunk][dk] query coefficient
  float* s_v = s_q + kChunk * dk;        // [kChunk][32] value column
  const int64_t row0 = a.seg_start[seg];
  const int n_vt = gridDim.x;
  float* st = a.state + (int64_t)a.seg_slot[seg] * a.state_slot_stride + ((int64_t)h * n_vt + vt) * (R * 256);
  float s[R];
#pragma unroll
  for (int i = 0; i < R; ++i) s[i] = st[i * 256 + tid];
  const int grp = SSD ? h / (a.heads / a.groups) : 0;
  const int inner = a.heads * a.dv;
  float skip = 0.f, neg_a = 0.f, dtb = 0.f;
  if (SSD) { skip = a.skip[h]; neg_a = -expf(a.a_log[h]); dtb = a.dt_bias[h]; }

  for (int t0 = 0; t0 < len; t0 += kChunk) {
    const int nt = min(kChunk, len - t0);
    __syncthreads();
    for (int i = tid; i < nt * dk; i += 256) {
      const int t = i / dk, d = i - t * dk;
      const int64_t r = row0 + t0 + t;
      if (SSD) {
        const float dt = softplus_f(a.P[r * a.ldp + a.off_dt + h] + dtb);
        s_a[i] = expf(neg_a * dt);
        s_k[i] = dt * a.xbc[r * a.ld_xbc + inner + grp * dk + d];
        s_q[i] = a.xbc[r * a.ld_xbc + inner + a.groups * dk + grp * dk + d];
      } else {
        const float zz = a.z[r * a.ldz + h * dk + d] + a.z_bias[h * dk + d];
        s_a[i] = expf(logsigmoid_f(zz) * a.inv_tau);
        s_k[i] = a.P[r * a.ldp + a.off_k + h * dk + d];
        s_q[i] = a.P[r * a.ldp + a.off_q + h * dk + d] * a.q_scale;
      }
    }
    for (int i = tid; i < nt * kColsPerCta; i += 256) {
      const int t = i / kColsPerCta, c = i - t * kColsPerCta;
      const int vv = vt * kColsPerCta + c;
      const int64_t r = row0 + t0 + t;
      float x = 0.f;
      if (vv < a.dv) x = SSD ? a.xbc[r * a.ld_xbc + h * a.dv + vv] : a.P[r * a.ldp + a.off_v + h * a.dv + vv];
      s_v[i] = x;
    }
    __syncthreads();
    for (int t = 0; t < nt; ++t) {
      const float xv = s_v[t * kColsPerCta + vl];
      const float* pa = s_a + t * dk;
      const float* pk = s_k + t * dk;
      const float* pq = s_q + t * dk;
      float acc = 0.f;
#pragma unroll
      for (int i = 0; i < R; ++i) {
        const int d = dg + kKeyLanes * i;
        if (d < dk) {
          s[i] = fmaf(pa[d], s[i], pk[d] * xv);
          acc = fmaf(s[i], pq[d], acc);
        }
      }
      acc += __shfl_xor_sync(0xffffffffu, acc, 1);
      acc += __shfl_xor_sync(0xffffffffu, acc, 2);
      acc += __shfl_xor_sync(0xffffffffu, acc, 4);
      if (dg == 0 && v_ok) a.out[(row0 + t0 + t) * a.ld_out + h * a.dv + v] = acc + skip * xv;
    }
  }
#pragma unroll
  for (int i = 0; i < R; ++i) st[i * 256 + tid] = s[i];
}

template <bool SSD>
int launch_scan(const ScanArgs& a, int n_seg, cudaStream_t st) {
  const int r_need = (a.dk + kKeyLanes - 1) / kKeyLanes;
  dim3 grid((a.dv + kColsPerCta - 1) / kColsPerCta, a.heads, n_seg);
  const size_t smem = (size_t)kChunk * (3 * a.dk + kColsPerCta) * sizeof(float);
  if (r_need <= 1) lin_scan_kernel<1, SSD><<<grid, 256, smem, st>>>(a);
  else if (r_need <= 2) lin_scan_kernel<2, SSD><<<grid, 256, smem, st>>>(a);
  else if (r_need <= 4) lin_scan_kernel<4, SSD><<<grid, 256, smem, st>>>(a);
  else if (r_need <= 8) lin_scan_kernel<8, SSD><<<grid, 256, smem, st>>>(a);
  else if (r_need <= 16) lin_scan_kernel<16, SSD><<<grid, 256, smem, st>>>(a);
  else lin_scan_kernel<32, SSD><<<grid, 256, smem, st>>>(a);
  PRL_LAUNCH_CHECK();
  return PRL_OK;
}

int scan_r(int dk) {
  const int need = (dk + kKeyLanes - 1) / kKeyLanes;
  int r = 1;
  while (r < need) r *= 2;
  return r;
}

}  // namespace
}  // namespace prl

using namespace prl;

extern "C" int64_t prl_lin_scan_state_floats(int32_t heads, int32_t dk, int32_t dv) {
  if (heads < 1 || dk < 1 || dk > 256 || dv < 1) return -1;
  const int64_t tiles = (dv + kColsPerCta - 1) / kColsPerCta;
  return (int64_t)heads * tiles * scan_r(dk) * 256;
}

extern "C" int prl_gla_scan(const float* P, int64_t ldp, int32_t off_q, int32_t off_k, int32_t off_v, float q_scale,
                            const float* z, int64_t ldz, const float* z_bias, float tau, int32_t heads, int32_t dk,
                            int32_t dv, const int32_t* seg_start, const int32_t* seg_len, const int32_t* seg_slot,
                            int32_t n_seg, float* state, float* out, int64_t ld_out, prl_stream_t st) {
  PRL_CHECK_ARG(P && z && z_bias && seg_start && seg_len && seg_slot && state && out, "prl_gla_scan: NULL argument");
  PRL_CHECK_ARG(heads >= 1 && dk >= 1 && dk <= 256 && dv >= 1 && n_seg >= 1 && n_seg <= 65535 && tau > 0.f,
                "prl_gla_scan: bad shape (heads=%d dk=%d dv=%d, dk at most 256)", heads, dk, dv);
  ScanArgs a = {};
  a.seg_start = seg_start; a.seg_len = seg_len; a.seg_slot = seg_slot;
  a.heads = heads; a.dk = dk; a.dv = dv;
  a.state = state; a.state_slot_stride = prl_lin_scan_state_floats(heads, dk, dv);
  a.out = out; a.ld_out = ld_out;
  a.P = P; a.ldp = ldp; a.off_q = off_q; a.off_k = off_k; a.off_v = off_v; a.q_scale = q_scale;
  a.z = z; a.ldz = ldz; a.z_bias = z_bias; a.inv_tau = 1.f / tau;
  return launch_scan<false>(a, n_seg, (cudaStream_t)st);
}

extern "C" int prl_ssd_scan(const float* P, int64_t ldp, int32_t off_dt, const float* xbc, int64_t ld_xbc,
                            const float* dt_bias, const float* a_log, const float* skip, int32_t heads, int32_t groups,
                            int32_t n_state, int32_t dv, const int32_t* seg_start, const int32_t* seg_len,
                            const int32_t* seg_slot, int32_t n_seg, float* state, float* out, int64_t ld_out,
                            prl_stream_t st) {
  PRL_CHECK_ARG(P && xbc && dt_bias && a_log && skip && seg_start && seg_len && seg_slot && state && out,
                "prl_ssd_scan: NULL argument");
  PRL_CHECK_ARG(heads >= 1 && groups >= 1 && heads % groups == 0 && n_state >= 1 && n_state <= 256 && dv >= 1 &&
                n_seg >= 1 && n_seg <= 65535,
                "prl_ssd_scan: bad shape (heads=%d groups=%d state=%d dv=%d, state at most 256)", heads, groups, n_state, dv);
  ScanArgs a = {};
  a.seg_start = seg_start; a.seg_len = seg_len; a.seg_slot = seg_slot;
  a.heads = heads; a.dk = n_state; a.dv = dv;
  a.state = state; a.state_slot_stride = prl_lin_scan_state_floats(heads, n_state, dv);
  a.out = out; a.ld_out = ld_out;
  a.P = P; a.ldp = ldp; a.off_dt = off_dt;
  a.xbc = xbc; a.ld_xbc = ld_xbc; a.groups = groups;
  a.dt_bias = dt_bias; a.a_log = a_log; a.skip = skip;
  return launch_scan<true>(a, n_seg, (cudaStream_t)st);
}
