// Causal softmax attention over a paged KV cache for ANY head geometry: query/key size `dim` and value size `vdim`
// are independent run-time numbers (the tcgen05 kernels of attn_tc.cu / paged_attn.cu are built for 128 = 128), the
// softmax scale is a parameter, the cache element type is bf16 or fp32.  Ragged segments: a segment is q_len
// consecutive tokens of one sequence starting at position pos0 (a prompt chunk, or one decoded token); token i of the
// segment sees keys 0 .. pos0 + i of its sequence, all of which are already in the cache.
//
// CTA = 8 warps = 8 consecutive query rows of one (segment, query head); the CTA streams the sequence's keys in tiles of
// 32 through shared memory (converted to fp32), a warp scores one key per lane, keeps an fp32 online softmax for its
// row and accumulates vdim / 32 output channels per lane.  Key tiles start at absolute multiples of 32, so the
// summation order for a query never depends on how its prompt was chunked or batched.
//
// Options (all off at 0): `window` > 0 hides keys more than window - 1 positions back, except the first `keep_first`
// tokens of the sequence, which every later token keeps seeing; `softcap` > 0 replaces a score s by
// softcap * tanh(s / softcap) before the softmax.  Key tiles that no row of the CTA can see are skipped whole, the
// others keep their absolute place, so the order of summation still does not depend on the chunking.  The output is
// fp32, or the cache's element type when out_is_t is set (it then feeds a GEMM directly).
//
// K pool: [page][kv head][page_size][dim], V pool: [page][kv head][page_size][vdim]; block_table[slot][j] = j-th page.
#include "prl_common.cuh"
#include <math.h>

namespace prl {
namespace {

constexpr int kRowsPerCta = 8;
constexpr int kKeysPerTile = 32;

template <typename T> __device__ __forceinline__ float cvt(T v);
template <> __device__ __forceinline__ float cvt<float>(float v) { return v; }
template <> __device__ __forceinline__ float cvt<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T, int VR, bool OUT_T>
__global__ void __launch_bounds__(256) attn_any_kernel(const T* __restrict__ q, const T* __restrict__ k_pool,
                                                       const T* __restrict__ v_pool, const int32_t* __restrict__ block_table,
                                                       int max_blocks, int page_size, const int32_t* __restrict__ seg_start,
                                                       const int32_t* __restrict__ seg_len, const int32_t* __restrict__ seg_pos0,
                                                       const int32_t* __restrict__ seg_slot, int H, int G, int dim, int vdim,
                                                       float scale, int window, int keep_first, float softcap,
                                                       void* __restrict__ out_v) {
  pdl_wait();   // launched with the programmatic-serialization attribute like the engine's other step kernels; no early
                // trigger: letting the next grid become resident early measured +3 ms on a 4096-token prefill and +-0 on decode
  extern __shared__ float sm[];
  const int seg = blockIdx.z, h = blockIdx.y, tile = blockIdx.x;
  const int len = seg_len[seg];
  const int i0 = tile * kRowsPerCta;
  if (i0 >= len) return;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = h / (H / G);
  const int slot = seg_slot[seg], pos0 = seg_pos0[seg];
  const int64_t row0 = seg_start[seg];
  const int kstride = dim + 1;
  float* Ks = sm;                                  // [32][dim + 1]
  float* Vs = Ks + kKeysPerTile * kstride;         // [32][vdim]
  float* Qs = Vs + kKeysPerTile * vdim;            // [8][dim]
  const int my_i = i0 + warp;
  const bool row_ok = my_i < len;
  const int my_pos = pos0 + my_i;
  const int rows_here = min(kRowsPerCta, len - i0);
  const int last_pos = pos0 + i0 + rows_here - 1;  // the CTA needs keys 0 .. last_pos
  // keys the CTA's FIRST row no longer sees end before win_lo; tiles wholly inside [sink_end, win_lo) are skipped
  const int win_lo = window > 0 ? max(0, pos0 + i0 - window + 1) : 0;
  const int sink_end = window > 0 ? min(keep_first, win_lo) : 0;
  const int my_lo = window > 0 ? my_pos - window + 1 : 0;     // this row sees j >= my_lo, and j < keep_first
  for (int i = threadIdx.x; i < rows_here * dim; i += blockDim.x) {
    const int w = i / dim, d = i - w * dim;
    Qs[w * dim + d] = cvt(q[((row0 + i0 + w) * H + h) * dim + d]);
  }
  float m = -INFINITY, l = 0.f;
  float acc[VR];
#pragma unroll
  for (int i = 0; i < VR; ++i) acc[i] = 0.f;
  const int32_t* bt = block_table + (int64_t)slot * max_blocks;
  for (int k0 = 0; k0 <= last_pos; k0 += kKeysPerTile) {
    if (k0 >= sink_end && k0 + kKeysPerTile <= win_lo) continue;     // CTA-uniform
    __syncthreads();
    const int nk = min(kKeysPerTile, last_pos + 1 - k0);
    for (int i = threadIdx.x; i < nk * dim; i += blockDim.x) {
      const int j = i / dim, d = i - j * dim;
      const int kt = k0 + j;
      const int page = bt[kt / page_size], within = kt % page_size;
      Ks[j * kstride + d] = cvt(k_pool[(((int64_t)page * G + g) * page_size + within) * dim + d]);
    }
    for (int i = threadIdx.x; i < nk * vdim; i += blockDim.x) {
      const int j = i / vdim, d = i - j * vdim;
      const int kt = k0 + j;
      const int page = bt[kt / page_size], within = kt % page_size;
      Vs[j * vdim + d] = cvt(v_pool[(((int64_t)page * G + g) * page_size + within) * vdim + d]);
    }
    __syncthreads();
    if (!row_ok || k0 > my_pos) continue;          // warp-uniform
    if (k0 + nk <= my_lo && k0 >= keep_first) continue;   // nothing of this tile is visible to this row (warp-uniform)
    float s = -INFINITY;
    const int kt_mine = k0 + lane;
    if (lane < nk && kt_mine <= my_pos && (kt_mine >= my_lo || kt_mine < keep_first)) {
      const float* qr = Qs + warp * dim;
      const float* kr = Ks + lane * kstride;
      float dot = 0.f;
      for (int d = 0; d < dim; ++d) dot = fmaf(qr[d], kr[d], dot);
      s = dot * scale;
      if (softcap > 0.f) s = softcap * tanhf(s / softcap);
    }
    const float m_new = fmaxf(m, warp_max(s));     // at least one key of the tile is visible, so m_new is finite
    const float corr = expf(m - m_new);            // exp(-inf) = 0 on the first tile
    const float p = (s == -INFINITY) ? 0.f : expf(s - m_new);
    l = l * corr + warp_sum(p);
    m = m_new;
#pragma unroll
    for (int i = 0; i < VR; ++i) acc[i] *= corr;
    const int n_vis = min(nk, my_pos - k0 + 1);
    for (int j = 0; j < n_vis; ++j) {
      const float pj = __shfl_sync(0xffffffffu, p, j);
      if (pj == 0.f) continue;                      // hidden key (warp-uniform)
#pragma unroll
      for (int i = 0; i < VR; ++i) {
        const int c = lane + 32 * i;
        if (c < vdim) acc[i] = fmaf(pj, Vs[j * vdim + c], acc[i]);
      }
    }
  }
  if (row_ok) {
    const float inv = 1.f / l;
#pragma unroll
    for (int i = 0; i < VR; ++i) {
      const int c = lane + 32 * i;
      if (c < vdim) {
        if constexpr (OUT_T) reinterpret_cast<T*>(out_v)[((row0 + my_i) * H + h) * vdim + c] = T(acc[i] * inv);
        else reinterpret_cast<float*>(out_v)[((row0 + my_i) * H + h) * vdim + c] = acc[i] * inv;
      }
    }
  }
}

template <typename T, int VR, bool OUT_T>
int launch_attn(const void* q, const void* kp, const void* vp, const int32_t* bt, int max_blocks, int page_size,
                const int32_t* ss, const int32_t* sl, const int32_t* sp, const int32_t* sslot, int n_seg, int max_q, int H,
                int G, int dim, int vdim, float scale, int window, int keep_first, float softcap, void* out, cudaStream_t st) {
  const size_t smem = ((size_t)kKeysPerTile * (dim + 1) + (size_t)kKeysPerTile * vdim + (size_t)kRowsPerCta * dim) * sizeof(float);
  static SmemAttr attr = {};
  if (smem > 48 * 1024) PRL_CUDA(ensure_smem(attn_any_kernel<T, VR, OUT_T>, (int)smem, attr));
  dim3 grid((max_q + kRowsPerCta - 1) / kRowsPerCta, H, n_seg);
  PRL_CUDA(launch_pdl((attn_any_kernel<T, VR, OUT_T>), dim3(grid), dim3(256), (size_t)(smem), st, (const T*)q, (const T*)kp, (const T*)vp, bt, max_blocks, page_size, ss, sl,
                      sp, sslot, H, G, dim, vdim, scale, window, keep_first, softcap, out));
  PRL_LAUNCH_CHECK();
  return PRL_OK;
}

template <typename T>
int dispatch_attn(int vr, const void* q, const void* kp, const void* vp, const int32_t* bt, int max_blocks, int page_size,
                  const int32_t* ss, const int32_t* sl, const int32_t* sp, const int32_t* sslot, int n_seg, int max_q, int H,
                  int G, int dim, int vdim, float scale, int window, int keep_first, float softcap, int out_is_t, void* out, cudaStream_t st) {
#define PRL_ATTN(VR) (out_is_t ? launch_attn<T, VR, true>(q, kp, vp, bt, max_blocks, page_size, ss, sl, sp, sslot, n_seg, max_q, H, G, dim, vdim, scale, window, keep_first, softcap, out, st) \
                               : launch_attn<T, VR, false>(q, kp, vp, bt, max_blocks, page_size, ss, sl, sp, sslot, n_seg, max_q, H, G, dim, vdim, scale, window, keep_first, softcap, out, st))
  if (vr <= 1) return PRL_ATTN(1);
  if (vr <= 2) return PRL_ATTN(2);
  if (vr <= 4) return PRL_ATTN(4);
  return PRL_ATTN(8);
#undef PRL_ATTN
}

}  // namespace
}  // namespace prl

using namespace prl;

static int attn_any_impl(const void* q, const void* k_pool, const void* v_pool, int32_t f32, const int32_t* block_table,
                         int32_t max_blocks, int32_t page_size, const int32_t* seg_start, const int32_t* seg_len,
                         const int32_t* seg_pos0, const int32_t* seg_slot, int32_t n_seg, int32_t max_q, int32_t H,
                         int32_t G, int32_t dim, int32_t vdim, float scale, int32_t window, int32_t keep_first,
                         float softcap, int32_t out_is_t, void* out, prl_stream_t st) {
  PRL_CHECK_ARG(q && k_pool && v_pool && block_table && seg_start && seg_len && seg_pos0 && seg_slot && out,
                "prl_attn_any: NULL argument");
  PRL_CHECK_ARG(n_seg >= 1 && n_seg <= 65535 && max_q >= 1 && H >= 1 && H <= 65535 && G >= 1 && H % G == 0 && dim >= 1 &&
                dim <= 512 && vdim >= 1 && vdim <= 256 && page_size >= 1 && max_blocks >= 1,
                "prl_attn_any: bad shape (H=%d G=%d dim=%d vdim=%d; dim <= 512, vdim <= 256)", H, G, dim, vdim);
  PRL_CHECK_ARG(window >= 0 && keep_first >= 0 && softcap >= 0.f, "prl_attn_any: bad mask (window=%d keep_first=%d)", window, keep_first);
  const int vr = (vdim + 31) / 32;
  if (f32) return dispatch_attn<float>(vr, q, k_pool, v_pool, block_table, max_blocks, page_size, seg_start, seg_len, seg_pos0,
                                       seg_slot, n_seg, max_q, H, G, dim, vdim, scale, window, keep_first, softcap, out_is_t, out, (cudaStream_t)st);
  return dispatch_attn<__nv_bfloat16>(vr, q, k_pool, v_pool, block_table, max_blocks, page_size, seg_start, seg_len, seg_pos0,
                                      seg_slot, n_seg, max_q, H, G, dim, vdim, scale, window, keep_first, softcap, out_is_t, out, (cudaStream_t)st);
}

extern "C" int prl_attn_any(const void* q, const void* k_pool, const void* v_pool, int32_t f32, const int32_t* block_table,
                            int32_t max_blocks, int32_t page_size, const int32_t* seg_start, const int32_t* seg_len,
                            const int32_t* seg_pos0, const int32_t* seg_slot, int32_t n_seg, int32_t max_q, int32_t H,
                            int32_t G, int32_t dim, int32_t vdim, float scale, float* out, prl_stream_t st) {
  return attn_any_impl(q, k_pool, v_pool, f32, block_table, max_blocks, page_size, seg_start, seg_len, seg_pos0, seg_slot,
                       n_seg, max_q, H, G, dim, vdim, scale, 0, 0, 0.f, 0, out, st);
}

// With a sliding window (0 = none) that keeps the first `keep_first` tokens, a tanh cap on the scores (0 = none) and
// the output in the cache's element type (out_is_t) or fp32.
extern "C" int prl_attn_any_masked(const void* q, const void* k_pool, const void* v_pool, int32_t f32,
                                   const int32_t* block_table, int32_t max_blocks, int32_t page_size,
                                   const int32_t* seg_start, const int32_t* seg_len, const int32_t* seg_pos0,
                                   const int32_t* seg_slot, int32_t n_seg, int32_t max_q, int32_t H, int32_t G, int32_t dim,
                                   int32_t vdim, float scale, int32_t window, int32_t keep_first, float softcap,
                                   int32_t out_is_t, void* out, prl_stream_t st) {
  return attn_any_impl(q, k_pool, v_pool, f32, block_table, max_blocks, page_size, seg_start, seg_len, seg_pos0, seg_slot,
                       n_seg, max_q, H, G, dim, vdim, scale, window, keep_first, softcap, out_is_t, out, st);
}
