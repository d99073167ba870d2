// Linear recurrences with a matrix state per head, over ragged rows:
//
//     S_t = diag(a_t) S_(t-1) + k_t v_t^T          S: [dk, dv]  (fp32, carried per sequence slot)
//     o_t = S_t^T q_t  (+ skip * v_t)
//
// Two front ends feed the same recurrence:
//   GATED  gated linear attention: q, k, v are columns of the projection buffer, the decay a_t is a vector per key
//          channel, a = sigmoid(z + bias)^(1/tau), formed beforehand by prl_gla_decay as exp(logsigmoid(z + bias) / tau),
//          and the output is scaled by q_scale;
//   SSD    state-space duality (Mamba-2): v = x (convolved), k = dt * B, q = C, the decay is one scalar per head,
//          a = exp(-exp(A_log) * dt) with dt = softplus(dt_raw + dt_bias), and skip = D.
//   SCALAR one decay and one input scale per head and token, S_t = a_t S_(t-1) + b_t k_t v_t^T: either a constant decay per
//          head with b = 1 (lightning attention) or (a_t, b_t) pairs formed beforehand (the stabilised exponential gates
//          of a matrix-memory LSTM, prl_mlstm_gates); q, k, v are columns of the projection buffer, the output is scaled
//          by q_scale.
// Everything that enters the recurrence is fp32.
//
// Work split: grid (value tiles, heads, segments), 64 threads per CTA.  Thread t owns VC adjacent value columns
// (t / 8) * VC .. and the key channels d = (t % 8) * R .. + R - 1, i.e. R x VC state elements in registers; a, k, q
// of a token are read from shared memory once per key channel and reused for the VC columns (128-bit loads from a
// padded, conflict-free layout); the 8 partial dot products of a column are summed with three shuffles.  VC (4, 2
// or 1) is picked per launch so that the grid fills the SMs: many sequences take wide tiles (a, k, q staged once per
// 32 columns), a single long prompt takes narrow ones (four times as many CTAs).  The arithmetic per state element
// is the same for every VC, bit for bit.  A CTA walks
// its segment token by token; tokens are staged kChunk at a time with cp.async into a double buffer, so the loads of
// the next chunk overlap the arithmetic of this one.  Prefill of a chunk and a single decoded token are the same
// code: a decode step is a segment of length 1 whose cost is the state's round trip through HBM.  The state is stored
// as [slot][head][r][column / 4][key lane][column % 4], which a warp reads as whole 128-byte lines for every VC; the layout
// is private to this file.  The result for a token depends only on the tokens before it in its own sequence: chunk
// borders, batch composition and slot numbers cannot change a bit of it.
#include "prl_common.cuh"

namespace prl {
namespace {

constexpr int kChunk = 8;       // tokens staged per round
constexpr int kKeyLanes = 8;    // threads that share a value column
constexpr int kThreads = 64;

struct ScanArgs {
  const int32_t* seg_start; const int32_t* seg_len; const int32_t* seg_slot;
  int heads, dk, dv;
  float* state; int64_t state_slot_stride;      // floats per slot
  float* out; int64_t ld_out;                   // [n, heads*dv] fp32
  // per-token vectors: base + row * ld + column offset (the head / group offset is added in the kernel)
  const float* kvec; int64_t ld_k; int off_k;
  const float* qvec; int64_t ld_q; int off_q;
  const float* avec; int64_t ld_a;              // GATED: decay per key channel
  const float* xval; int64_t ld_x; int off_x;   // value columns
  float q_scale;
  // SSD scalars
  const float* dt_raw; int64_t ld_dt; int off_dt; int groups;
  const float* dt_bias; const float* a_log; const float* skip;
  int vec4;   // every staged vector starts on a 16-byte boundary and dk, dv are multiples of 4: 16-byte cp.async
  // SCALAR: (decay, input scale) pairs at dt_raw[row * ld_dt + off_dt + 2 * head], or, if dt_raw is null, the constant
  // decay a_log[head] with input scale 1
  int zero_init;   // the state starts at zero instead of being read (seg_slot may then be null: slot = segment index)
};

__device__ __forceinline__ float softplus_f(float x) { return fmaxf(x, 0.f) + log1pf(expf(-fabsf(x))); }
__device__ __forceinline__ float logsigmoid_f(float x) { return fminf(x, 0.f) - log1pf(expf(-fabsf(x))); }

__device__ __forceinline__ void cp_async4(float* dst, const float* src) {
  const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(d), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async16(float* dst, const float* src) {
  const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

constexpr int kGated = 0, kSsd = 1, kScalar = 2;

template <int R, int VC, int MODE>
__global__ void __launch_bounds__(kThreads) lin_scan_kernel(ScanArgs a) {
  constexpr bool SSD = MODE == kSsd, SCL = MODE == kScalar, ONE = SSD || SCL;   // ONE: one decay per head and token
  pdl_wait();   // launched with the programmatic-serialization attribute like the engine's other step kernels; no early
                // trigger: letting the next grid become resident early measured +3 ms on a 4096-token prefill and +-0 on decode
  constexpr int kCols = kKeyLanes * VC;          // value columns per CTA
  constexpr int RS = R + 4;                      // padded stride of one thread's key-channel block (conflict-free LDS.128)
  constexpr int kVecTok = kKeyLanes * RS;        // floats per token and vector
  constexpr int kNVec = ONE ? 2 : 3;
  constexpr int kBuf = kChunk * (kNVec * kVecTok + kCols + 2);
  extern __shared__ __align__(16) float sm[];
  const int seg = blockIdx.z, h = blockIdx.y, vt = blockIdx.x;
  const int len = a.seg_len[seg];
  if (len <= 0) return;
  const int tid = threadIdx.x, dg = tid % kKeyLanes, vg = tid / kKeyLanes;
  const int dk = a.dk, dv = a.dv;
  const int64_t row0 = a.seg_start[seg];
  const int nv4 = (dv + 3) / 4;                  // state layout: [head][r][column / 4][key lane][column % 4]
  const int slot = a.seg_slot ? a.seg_slot[seg] : seg;
  float* st = a.state + (int64_t)slot * a.state_slot_stride + (int64_t)h * R * nv4 * 32;
  const int col0 = vt * kCols + vg * VC;
  float s[R][VC];
#pragma unroll
  for (int i = 0; i < R; ++i) {
    if constexpr (VC == 4) {        // col0 is a multiple of 4: the thread's four columns are one 16-byte group
      float4 v4 = make_float4(0.f, 0.f, 0.f, 0.f);
      if (col0 < nv4 * 4 && !a.zero_init)
        v4 = *reinterpret_cast<const float4*>(st + (((int64_t)i * nv4 + col0 / 4) * kKeyLanes + dg) * 4);
      s[i][0] = v4.x; s[i][1] = v4.y; s[i][2] = v4.z; s[i][3] = v4.w;
    } else {
#pragma unroll
      for (int j = 0; j < VC; ++j) {
        const int c = col0 + j;
        s[i][j] = (c < nv4 * 4 && !a.zero_init) ? st[(((int64_t)i * nv4 + c / 4) * kKeyLanes + dg) * 4 + (c & 3)] : 0.f;
      }
    }
  }
  const int grp = SSD ? h / (a.heads / a.groups) : 0;
  float skip = 0.f, neg_a = 0.f, dtb = 0.f;
  if (SSD) { skip = a.skip[h]; neg_a = -expf(a.a_log[h]); dtb = a.dt_bias[h]; }
  const float cdec = (SCL && !a.dt_raw) ? a.a_log[h] : 0.f;
  for (int i = tid; i < 2 * kBuf; i += kThreads) sm[i] = 0.f;   // padding slots (d >= dk, v >= dv) stay zero for good
  __syncthreads();

  const float* kbase = a.kvec + a.off_k + (SSD ? grp : h) * dk;
  const float* qbase = a.qvec + a.off_q + (SSD ? grp : h) * dk;
  const float* abase = ONE ? nullptr : a.avec + h * dk;
  const float* xbase = a.xval + a.off_x + h * dv + vt * kCols;
  const int cols_here = min(kCols, dv - vt * kCols);

  auto stage = [&](int t0, float* buf) {
    const int nt = min(kChunk, len - t0);
    float* bk = buf;
    float* bq = bk + kChunk * kVecTok;
    float* ba = bq + kChunk * kVecTok;                       // GATED only
    float* bx = buf + kChunk * kNVec * kVecTok;
    float* bs = bx + kChunk * kCols;                         // SSD: raw dt per token
    if (R % 4 == 0 && a.vec4) {     // four key channels of one thread's block per copy
      for (int t = 0; t < nt; ++t) {
        const int64_t r = row0 + t0 + t;
        for (int d = tid * 4; d < dk; d += kThreads * 4) {
          const int o = t * kVecTok + (d / R) * RS + (d % R);
          cp_async16(bk + o, kbase + r * a.ld_k + d);
          cp_async16(bq + o, qbase + r * a.ld_q + d);
          if (!ONE) cp_async16(ba + o, abase + r * a.ld_a + d);
        }
      }
      for (int i = tid * 4; i < nt * kCols; i += kThreads * 4) {
        const int t = i / kCols, c = i % kCols;
        if (c < cols_here) cp_async16(bx + t * kCols + c, xbase + (row0 + t0 + t) * a.ld_x + c);
      }
    } else {
      for (int t = 0; t < nt; ++t) {
        const int64_t r = row0 + t0 + t;
        for (int d = tid; d < dk; d += kThreads) {
          const int o = t * kVecTok + (d / R) * RS + (d % R);
          cp_async4(bk + o, kbase + r * a.ld_k + d);
          cp_async4(bq + o, qbase + r * a.ld_q + d);
          if (!ONE) cp_async4(ba + o, abase + r * a.ld_a + d);
        }
      }
      for (int i = tid; i < nt * kCols; i += kThreads) {
        const int t = i / kCols, c = i % kCols;
        if (c < cols_here) cp_async4(bx + t * kCols + c, xbase + (row0 + t0 + t) * a.ld_x + c);
      }
    }
    if (SSD && tid < nt) cp_async4(bs + tid, a.dt_raw + (row0 + t0 + tid) * a.ld_dt + a.off_dt + h);
    if (SCL && a.dt_raw && tid < nt) {
      const float* gp = a.dt_raw + (row0 + t0 + tid) * a.ld_dt + a.off_dt + 2 * h;
      cp_async4(bs + kChunk + tid, gp);      // decay
      cp_async4(bs + tid, gp + 1);           // input scale
    }
    cp_async_commit();
  };

  stage(0, sm);
  int cur = 0;
  for (int t0 = 0; t0 < len; t0 += kChunk, cur ^= 1) {
    const int nt = min(kChunk, len - t0);
    float* buf = sm + cur * kBuf;
    if (t0 + kChunk < len) {
      stage(t0 + kChunk, sm + (cur ^ 1) * kBuf);
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    const float* bk = buf;
    const float* bq = bk + kChunk * kVecTok;
    const float* ba = bq + kChunk * kVecTok;
    const float* bx = buf + kChunk * kNVec * kVecTok;
    float* bs = buf + kChunk * kNVec * kVecTok + kChunk * kCols;
    if (SSD) {
      if (tid < nt) {
        const float dt = softplus_f(bs[tid] + dtb);
        bs[tid] = dt;
        bs[kChunk + tid] = expf(neg_a * dt);
      }
      __syncthreads();
    }
    if (SCL && !a.dt_raw) {
      if (tid < nt) { bs[tid] = 1.f; bs[kChunk + tid] = cdec; }
      __syncthreads();
    }
    auto token = [&](int t) {
      float xv[VC], xin[VC], acc[VC];
#pragma unroll
      for (int j = 0; j < VC; ++j) {
        xv[j] = bx[t * kCols + vg * VC + j];
        xin[j] = ONE ? xv[j] * bs[t] : xv[j];
        acc[j] = 0.f;
      }
      const float dec = ONE ? bs[kChunk + t] : 0.f;
      const float* pk = bk + t * kVecTok + dg * RS;
      const float* pq = bq + t * kVecTok + dg * RS;
      const float* pa = ba + t * kVecTok + dg * RS;
      if constexpr (R % 4 == 0) {
#pragma unroll
        for (int i4 = 0; i4 < R / 4; ++i4) {
          const float4 k4 = *reinterpret_cast<const float4*>(pk + 4 * i4);
          const float4 q4 = *reinterpret_cast<const float4*>(pq + 4 * i4);
          float4 a4 = make_float4(dec, dec, dec, dec);
          if (!ONE) a4 = *reinterpret_cast<const float4*>(pa + 4 * i4);
          const float kk[4] = {k4.x, k4.y, k4.z, k4.w}, qq[4] = {q4.x, q4.y, q4.z, q4.w}, aa[4] = {a4.x, a4.y, a4.z, a4.w};
#pragma unroll
          for (int u = 0; u < 4; ++u)
#pragma unroll
            for (int j = 0; j < VC; ++j) {
              s[4 * i4 + u][j] = fmaf(aa[u], s[4 * i4 + u][j], kk[u] * xin[j]);
              acc[j] = fmaf(s[4 * i4 + u][j], qq[u], acc[j]);
            }
        }
      } else {
#pragma unroll
        for (int i = 0; i < R; ++i) {
          const float kk = pk[i], qq = pq[i], aa = ONE ? dec : pa[i];
#pragma unroll
          for (int j = 0; j < VC; ++j) {
            s[i][j] = fmaf(aa, s[i][j], kk * xin[j]);
            acc[j] = fmaf(s[i][j], qq, acc[j]);
          }
        }
      }
#pragma unroll
      for (int j = 0; j < VC; ++j) {
        acc[j] += __shfl_xor_sync(0xffffffffu, acc[j], 1);
        acc[j] += __shfl_xor_sync(0xffffffffu, acc[j], 2);
        acc[j] += __shfl_xor_sync(0xffffffffu, acc[j], 4);
      }
      if (dg == 0) {
        float* o = a.out + (row0 + t0 + t) * a.ld_out + h * dv + vt * kCols + vg * VC;
#pragma unroll
        for (int j = 0; j < VC; ++j)
          if (vg * VC + j < cols_here) o[j] = SSD ? acc[j] + skip * xv[j] : acc[j] * a.q_scale;
      }
    };
    if (nt == kChunk) {   // a full chunk: unrolled, so that one token's shuffles and store overlap the next token's loads
#pragma unroll
      for (int t = 0; t < kChunk; ++t) token(t);
    } else {
      for (int t = 0; t < nt; ++t) token(t);
    }
    __syncthreads();     // the buffer is free for the chunk after next
  }
#pragma unroll
  for (int i = 0; i < R; ++i) {
    if constexpr (VC == 4) {
      if (col0 < nv4 * 4)
        *reinterpret_cast<float4*>(st + (((int64_t)i * nv4 + col0 / 4) * kKeyLanes + dg) * 4) =
            make_float4(s[i][0], s[i][1], s[i][2], s[i][3]);
    } else {
#pragma unroll
      for (int j = 0; j < VC; ++j) {
        const int c = col0 + j;
        if (c < nv4 * 4) st[(((int64_t)i * nv4 + c / 4) * kKeyLanes + dg) * 4 + (c & 3)] = s[i][j];
      }
    }
  }
}

// R = key channels per thread (dk <= 8 R, a power of two)
int plan_r(int dk) {
  const int need = (dk + kKeyLanes - 1) / kKeyLanes;
  int r = 1;
  while (r < need) r *= 2;
  return r;
}

template <int R, int VC, int SSD>
int launch_one(const ScanArgs& a, int n_seg, cudaStream_t st) {
  constexpr int kCols = kKeyLanes * VC;
  constexpr int kNVec = SSD != kGated ? 2 : 3;
  const size_t smem = 2 * (size_t)kChunk * (kNVec * kKeyLanes * (R + 4) + kCols + 2) * sizeof(float);
  static SmemAttr attr = {};
  if (smem > 48 * 1024) PRL_CUDA(ensure_smem(lin_scan_kernel<R, VC, SSD>, (int)smem, attr));
  dim3 grid((a.dv + kCols - 1) / kCols, a.heads, n_seg);
  PRL_CUDA(launch_pdl((lin_scan_kernel<R, VC, SSD>), dim3(grid), dim3(kThreads), (size_t)(smem), st, a));
  PRL_LAUNCH_CHECK();
  return PRL_OK;
}

// value columns per thread: the widest tile that still gives two CTAs per SM
template <int R, int SSD>
int launch_r(const ScanArgs& a, int n_seg, cudaStream_t st) {
  const int64_t want = 2 * (int64_t)num_sms();
  auto ctas = [&](int vc) { return (int64_t)((a.dv + 8 * vc - 1) / (8 * vc)) * a.heads * n_seg; };
  if (R <= 16 && ctas(4) >= want) return launch_one<R, (R <= 16 ? 4 : 2), SSD>(a, n_seg, st);
  if (ctas(2) >= want) return launch_one<R, 2, SSD>(a, n_seg, st);
  return launch_one<R, 1, SSD>(a, n_seg, st);
}

inline bool aligned16(const void* p) { return ((uintptr_t)p & 15) == 0; }

template <int SSD>
int launch_scan(ScanArgs a, int n_seg, cudaStream_t st) {
  a.vec4 = (a.dk % 4 == 0 && a.dv % 4 == 0 && a.ld_k % 4 == 0 && a.ld_q % 4 == 0 && a.ld_x % 4 == 0 && a.off_k % 4 == 0 &&
            a.off_q % 4 == 0 && a.off_x % 4 == 0 && aligned16(a.kvec) && aligned16(a.qvec) && aligned16(a.xval) &&
            (SSD != kGated || (a.ld_a % 4 == 0 && aligned16(a.avec)))) ? 1 : 0;
  switch (plan_r(a.dk)) {
    case 1: return launch_r<1, SSD>(a, n_seg, st);
    case 2: return launch_r<2, SSD>(a, n_seg, st);
    case 4: return launch_r<4, SSD>(a, n_seg, st);
    case 8: return launch_r<8, SSD>(a, n_seg, st);
    case 16: return launch_r<16, SSD>(a, n_seg, st);
    default: return launch_r<32, SSD>(a, n_seg, st);
  }
}

__global__ void gla_decay_kernel(float* __restrict__ z, int64_t ldz, const float* __restrict__ bias, float inv_tau, int C) {
  pdl_wait();
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= C) return;
  float* p = z + (int64_t)blockIdx.x * ldz + c;
  *p = expf(logsigmoid_f(*p + bias[c]) * inv_tau);
}


// ---- the same recurrences with a long segment cut into pieces that run side by side ---------------------------------
// A prompt portion of one sequence gives lin_scan_kernel only (value tiles x heads) CTAs, a fraction of a warp per
// scheduler, and the walk over its tokens is a dependent chain.  The recurrence is linear in the state, so a segment
// may be cut into pieces of at most kPiece tokens:
//   1. lin_scan_kernel runs every piece from a ZERO state (pieces are independent: pieces x heads x tiles CTAs); it
//      writes o_t^local and leaves the piece's own contribution L_c in a scratch state;
//   2. piece_decay_kernel: D_c[d] = prod of a_t[d] over the piece;
//   3. carry_kernel walks the pieces of a segment in order, per state element: scratch[c] <- S (the state BEFORE piece
//      c), S <- D_c * S + L_c; the last S is the sequence's new state;
//   4. apply_kernel adds what the incoming state contributes: o_t += (q_t * prod_{s <= t in piece} a_s)^T S_before(c),
//      a [tokens x dk] x [dk x dv] product per piece and head from shared memory.
// All of it is fp32; the result differs from the token-by-token walk by the rounding of a different summation order.
constexpr int kPiece = 64;          // tokens per piece at most (the token tile of apply_kernel)
constexpr int kApplyCols = 64;      // value columns per CTA of apply_kernel
constexpr int kApplyKeys = 64;      // key channels per round of apply_kernel
constexpr int kWStride = kPiece + 4;

struct SplitArgs {
  const int32_t* sub_start; const int32_t* sub_len;     // the pieces (rows of the batch); scratch slot = piece index
  const int32_t* seg_sub0; const int32_t* seg_nsub;      // first piece and piece count of every segment
  float* scratch;                                        // [pieces][state_slot_stride]
  float* cdec;                                           // [pieces][heads][8 r]
  int r;                                                 // key channels per key lane in the state layout
};

template <int MODE>
__global__ void __launch_bounds__(256) piece_decay_kernel(ScanArgs a, SplitArgs p) {
  constexpr bool SSD = MODE == kSsd, SCL = MODE == kScalar;
  pdl_wait();
  const int sub = blockIdx.x, h = blockIdx.y, d = threadIdx.x, dpad = kKeyLanes * p.r;
  if (d >= dpad) return;
  const int len = p.sub_len[sub];
  const int64_t row0 = p.sub_start[sub];
  float prod = 1.f;                    // eight loads in flight at a time; the product keeps the order of the tokens
  const float neg_a = SSD ? -expf(a.a_log[h]) : 0.f, dtb = SSD ? a.dt_bias[h] : 0.f;
  const float cdec = (SCL && !a.dt_raw) ? a.a_log[h] : 1.f;
  if (SSD || SCL || d < a.dk) {
    for (int t0 = 0; t0 < len; t0 += 8) {
      float v[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int t = min(t0 + j, len - 1);
        if (SCL) v[j] = a.dt_raw ? a.dt_raw[(row0 + t) * a.ld_dt + a.off_dt + 2 * h] : cdec;
        else v[j] = SSD ? a.dt_raw[(row0 + t) * a.ld_dt + a.off_dt + h] : a.avec[(row0 + t) * a.ld_a + h * a.dk + d];
      }
#pragma unroll
      for (int j = 0; j < 8; ++j)
        if (t0 + j < len) prod *= SSD ? expf(neg_a * softplus_f(v[j] + dtb)) : v[j];
    }
  }
  p.cdec[((int64_t)sub * a.heads + h) * dpad + d] = prod;
}

__global__ void __launch_bounds__(256) carry_kernel(ScanArgs a, SplitArgs p) {
  pdl_wait();
  const int seg = blockIdx.z, h = blockIdx.y;
  const int nv4 = (a.dv + 3) / 4, per_head = p.r * nv4 * 32, dpad = kKeyLanes * p.r;
  const int idx = (blockIdx.x * 256 + threadIdx.x) * 4;          // four columns of one key channel
  if (idx >= per_head) return;
  const int d = ((idx / 4) % kKeyLanes) * p.r + idx / (nv4 * 32);
  const int64_t off = (int64_t)h * per_head + idx;
  float4* real = reinterpret_cast<float4*>(a.state + (int64_t)a.seg_slot[seg] * a.state_slot_stride + off);
  float4 s = *real;
  const int sub0 = p.seg_sub0[seg], nsub = p.seg_nsub[seg];
  for (int c0 = 0; c0 < nsub; c0 += 8) {       // the loads of eight pieces are in flight together; the chain is arithmetic only
    float4 loc[8];
    float dc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int sub = sub0 + min(c0 + j, nsub - 1);
      dc[j] = p.cdec[((int64_t)sub * a.heads + h) * dpad + d];
      loc[j] = *reinterpret_cast<const float4*>(p.scratch + (int64_t)sub * a.state_slot_stride + off);
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      if (c0 + j < nsub) {
        *reinterpret_cast<float4*>(p.scratch + (int64_t)(sub0 + c0 + j) * a.state_slot_stride + off) = s;
        s = make_float4(fmaf(dc[j], s.x, loc[j].x), fmaf(dc[j], s.y, loc[j].y), fmaf(dc[j], s.z, loc[j].z),
                        fmaf(dc[j], s.w, loc[j].w));
      }
    }
  }
  *real = s;
}

template <int MODE>
__global__ void __launch_bounds__(256) apply_kernel(ScanArgs a, SplitArgs p) {
  constexpr bool SSD = MODE == kSsd, SCL = MODE == kScalar, ONE = SSD || SCL;
  pdl_wait();
  __shared__ __align__(16) float wT[kApplyKeys * kWStride];     // [key channel][token]: q_t[d] * (decay from the piece's start through t)
  __shared__ __align__(16) float S[kApplyKeys * kApplyCols];    // [key channel][column]: the state before this piece
  __shared__ float dec[kPiece];
  const int sub = blockIdx.x, h = blockIdx.y, vt = blockIdx.z, tid = threadIdx.x;
  const int len = p.sub_len[sub], dk = a.dk, dv = a.dv, r = p.r;
  const int64_t row0 = p.sub_start[sub];
  const int grp = SSD ? h / (a.heads / a.groups) : 0;
  const float* qbase = a.qvec + a.off_q + (SSD ? grp : h) * dk;
  const int nv4 = (dv + 3) / 4;
  const float* sc = p.scratch + (int64_t)sub * a.state_slot_stride + (int64_t)h * r * nv4 * 32;
  const int tx = tid % 16, ty = tid / 16;      // columns 4 tx .., tokens 4 ty ..
  float acc[4][4] = {};
  if (ONE) {
    if (tid < kPiece) {
      if (SSD) dec[tid] = tid < len ? expf(-expf(a.a_log[h]) * softplus_f(a.dt_raw[(row0 + tid) * a.ld_dt + a.off_dt + h] + a.dt_bias[h])) : 1.f;
      else dec[tid] = tid < len ? (a.dt_raw ? a.dt_raw[(row0 + tid) * a.ld_dt + a.off_dt + 2 * h] : a.a_log[h]) : 1.f;
    }
    __syncthreads();
    if (tid == 0) {
      float cum = 1.f;
      for (int t = 0; t < kPiece; ++t) { cum *= dec[t]; dec[t] = cum; }
    }
    __syncthreads();
  }
  // key channels in blocks of kApplyKeys.  Within a block: the decays of the piece, their running product over its
  // tokens, times q -- every global load independent of the others (a thread per channel walking the tokens would
  // wait for each load in turn) -- then the state rows of these channels, then the product.
  for (int d0 = 0; d0 < dk; d0 += kApplyKeys) {
    const int nd = min(kApplyKeys, dk - d0);
    if (!ONE) {
      for (int e = tid; e < kPiece * nd; e += 256) {
        const int t = e / nd, d = e - t * nd;
        wT[d * kWStride + t] = t < len ? a.avec[(row0 + t) * a.ld_a + h * dk + d0 + d] : 1.f;
      }
      __syncthreads();
      if (tid < nd) {
        float cum = 1.f;
#pragma unroll 16
        for (int t = 0; t < kPiece; ++t) { cum *= wT[tid * kWStride + t]; wT[tid * kWStride + t] = cum; }
      }
      __syncthreads();
    }
    for (int e = tid; e < kPiece * nd; e += 256) {
      const int t = e / nd, d = e - t * nd;
      const float cum = ONE ? dec[t] : wT[d * kWStride + t];
      wT[d * kWStride + t] = t < len ? cum * qbase[(row0 + t) * a.ld_q + d0 + d] * a.q_scale : 0.f;
    }
    for (int e = tid; e < r * (kApplyCols / 4) * kKeyLanes; e += 256) {      // key lanes fastest: whole 128-byte lines
      const int dg = e % kKeyLanes, c4 = (e / kKeyLanes) % (kApplyCols / 4), i = e / (kKeyLanes * (kApplyCols / 4));
      const int d = dg * r + i - d0, col4 = vt * (kApplyCols / 4) + c4;
      if (d < 0 || d >= nd) continue;
      float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
      if (col4 < nv4) v = *reinterpret_cast<const float4*>(sc + (((int64_t)i * nv4 + col4) * kKeyLanes + dg) * 4);
      *reinterpret_cast<float4*>(S + d * kApplyCols + c4 * 4) = v;
    }
    __syncthreads();
    if (ty * 4 < len) {
#pragma unroll 4
      for (int d = 0; d < nd; ++d) {
        const float4 w4 = *reinterpret_cast<const float4*>(wT + d * kWStride + ty * 4);
        const float4 s4 = *reinterpret_cast<const float4*>(S + d * kApplyCols + tx * 4);
        const float ww[4] = {w4.x, w4.y, w4.z, w4.w}, ss[4] = {s4.x, s4.y, s4.z, s4.w};
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
          for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(ww[i], ss[j], acc[i][j]);
      }
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int t = ty * 4 + i;
    if (t >= len) break;
    float* o = a.out + (row0 + t) * a.ld_out + h * dv + vt * kApplyCols + tx * 4;
#pragma unroll
    for (int j = 0; j < 4; ++j)
      if (vt * kApplyCols + tx * 4 + j < dv) o[j] += acc[i][j];
  }
}

template <int SSD>
int launch_split(ScanArgs a, int n_seg, SplitArgs p, int n_sub, cudaStream_t st) {
  p.r = plan_r(a.dk);
  ScanArgs pieces = a;                 // 1. every piece from a zero state into its scratch slot
  pieces.seg_start = p.sub_start; pieces.seg_len = p.sub_len; pieces.seg_slot = nullptr;
  pieces.state = p.scratch; pieces.zero_init = 1;
  const int rc = launch_scan<SSD>(pieces, n_sub, st);
  if (rc != PRL_OK) return rc;
  PRL_CUDA(launch_pdl(piece_decay_kernel<SSD>, dim3(n_sub, a.heads), dim3(256), (size_t)0, st, a, p));
  PRL_LAUNCH_CHECK();
  const int nv4 = (a.dv + 3) / 4, per_head = p.r * nv4 * 32;
  PRL_CUDA(launch_pdl(carry_kernel, dim3((per_head + 1023) / 1024, a.heads, n_seg), dim3(256), (size_t)0, st, a, p));
  PRL_LAUNCH_CHECK();
  PRL_CUDA(launch_pdl(apply_kernel<SSD>, dim3(n_sub, a.heads, (a.dv + kApplyCols - 1) / kApplyCols), dim3(256), (size_t)0, st, a, p));
  PRL_LAUNCH_CHECK();
  return PRL_OK;
}

}  // namespace
}  // namespace prl

using namespace prl;

extern "C" int64_t prl_lin_scan_state_floats(int32_t heads, int32_t dk, int32_t dv) {
  if (heads < 1 || dk < 1 || dk > 256 || dv < 1) return -1;
  return (int64_t)heads * plan_r(dk) * ((dv + 3) / 4) * 32;
}

extern "C" int prl_gla_decay(float* z, int64_t ldz, const float* bias, float tau, int32_t n, int32_t C, prl_stream_t st) {
  PRL_CHECK_ARG(z && bias && n >= 1 && C >= 1 && ldz >= C && tau > 0.f, "prl_gla_decay: bad argument");
  PRL_CUDA(launch_pdl(gla_decay_kernel, dim3(n, (C + 255) / 256), dim3(256), (size_t)(0), (cudaStream_t)st, z, ldz, bias, 1.f / tau, C));
  PRL_LAUNCH_CHECK();
  return PRL_OK;
}

static int gla_scan_impl(const float* P, int64_t ldp, int32_t off_q, int32_t off_k, int32_t off_v, float q_scale,
                         const float* decay, int64_t ld_decay, int32_t heads, int32_t dk, int32_t dv,
                         const int32_t* seg_start, const int32_t* seg_len, const int32_t* seg_slot, int32_t n_seg,
                         float* state, float* out, int64_t ld_out, const SplitArgs* split, int32_t n_sub, prl_stream_t st) {
  PRL_CHECK_ARG(P && decay && seg_start && seg_len && seg_slot && state && out, "prl_gla_scan: NULL argument");
  PRL_CHECK_ARG(heads >= 1 && dk >= 1 && dk <= 256 && dv >= 1 && n_seg >= 1 && n_seg <= 65535,
                "prl_gla_scan: bad shape (heads=%d dk=%d dv=%d, dk at most 256)", heads, dk, dv);
  ScanArgs a = {};
  a.seg_start = seg_start; a.seg_len = seg_len; a.seg_slot = seg_slot;
  a.heads = heads; a.dk = dk; a.dv = dv;
  a.state = state; a.state_slot_stride = prl_lin_scan_state_floats(heads, dk, dv);
  a.out = out; a.ld_out = ld_out;
  a.kvec = P; a.ld_k = ldp; a.off_k = off_k;
  a.qvec = P; a.ld_q = ldp; a.off_q = off_q;
  a.avec = decay; a.ld_a = ld_decay;
  a.xval = P; a.ld_x = ldp; a.off_x = off_v;
  a.q_scale = q_scale;
  if (split) return launch_split<kGated>(a, n_seg, *split, n_sub, (cudaStream_t)st);
  return launch_scan<kGated>(a, n_seg, (cudaStream_t)st);
}

extern "C" int prl_gla_scan(const float* P, int64_t ldp, int32_t off_q, int32_t off_k, int32_t off_v, float q_scale,
                            const float* decay, int64_t ld_decay, int32_t heads, int32_t dk, int32_t dv,
                            const int32_t* seg_start, const int32_t* seg_len, const int32_t* seg_slot, int32_t n_seg,
                            float* state, float* out, int64_t ld_out, prl_stream_t st) {
  return gla_scan_impl(P, ldp, off_q, off_k, off_v, q_scale, decay, ld_decay, heads, dk, dv, seg_start, seg_len, seg_slot,
                       n_seg, state, out, ld_out, nullptr, 0, st);
}

static bool split_args(SplitArgs& p, const int32_t* seg_sub0, const int32_t* seg_nsub, const int32_t* sub_start,
                       const int32_t* sub_len, int32_t n_sub, float* scratch, float* cdec) {
  if (!seg_sub0 || !seg_nsub || !sub_start || !sub_len || !scratch || !cdec || n_sub < 1 || n_sub > 65535) return false;
  if (((uintptr_t)scratch & 15) != 0) return false;
  p = SplitArgs{};
  p.seg_sub0 = seg_sub0; p.seg_nsub = seg_nsub; p.sub_start = sub_start; p.sub_len = sub_len;
  p.scratch = scratch; p.cdec = cdec;
  return true;
}

// Floats of the per-piece decay table for one piece (the scratch state of a piece is prl_lin_scan_state_floats).
extern "C" int64_t prl_lin_scan_piece_decay_floats(int32_t heads, int32_t dk) {
  if (heads < 1 || dk < 1 || dk > 256) return -1;
  return (int64_t)heads * kKeyLanes * plan_r(dk);
}
extern "C" int32_t prl_lin_scan_piece_tokens() { return kPiece; }

// The same result as prl_gla_scan up to fp32 rounding, with every segment cut into pieces (rows sub_start[i] ..
// + sub_len[i], at most prl_lin_scan_piece_tokens() each, in order; segment s owns pieces seg_sub0[s] .. + seg_nsub[s])
// that run side by side.  scratch: [n_sub][prl_lin_scan_state_floats], cdec: [n_sub][prl_lin_scan_piece_decay_floats].
extern "C" int prl_gla_scan_split(const float* P, int64_t ldp, int32_t off_q, int32_t off_k, int32_t off_v, float q_scale,
                                  const float* decay, int64_t ld_decay, int32_t heads, int32_t dk, int32_t dv,
                                  const int32_t* seg_slot, int32_t n_seg, const int32_t* seg_sub0, const int32_t* seg_nsub,
                                  const int32_t* sub_start, const int32_t* sub_len, int32_t n_sub, float* scratch,
                                  float* cdec, float* state, float* out, int64_t ld_out, prl_stream_t st) {
  SplitArgs p;
  PRL_CHECK_ARG(split_args(p, seg_sub0, seg_nsub, sub_start, sub_len, n_sub, scratch, cdec), "prl_gla_scan_split: bad piece tables");
  return gla_scan_impl(P, ldp, off_q, off_k, off_v, q_scale, decay, ld_decay, heads, dk, dv, sub_start, sub_len, seg_slot,
                       n_seg, state, out, ld_out, &p, n_sub, st);
}

static int ssd_scan_impl(const float* P, int64_t ldp, int32_t off_dt, const float* xbc, int64_t ld_xbc,
                         const float* dt_bias, const float* a_log, const float* skip, int32_t heads, int32_t groups,
                         int32_t n_state, int32_t dv, const int32_t* seg_start, const int32_t* seg_len,
                         const int32_t* seg_slot, int32_t n_seg, float* state, float* out, int64_t ld_out,
                         const SplitArgs* split, int32_t n_sub, prl_stream_t st) {
  PRL_CHECK_ARG(P && xbc && dt_bias && a_log && skip && seg_start && seg_len && seg_slot && state && out,
                "prl_ssd_scan: NULL argument");
  PRL_CHECK_ARG(heads >= 1 && groups >= 1 && heads % groups == 0 && n_state >= 1 && n_state <= 256 && dv >= 1 &&
                n_seg >= 1 && n_seg <= 65535,
                "prl_ssd_scan: bad shape (heads=%d groups=%d state=%d dv=%d, state at most 256)", heads, groups, n_state, dv);
  const int inner = heads * dv;
  ScanArgs a = {};
  a.seg_start = seg_start; a.seg_len = seg_len; a.seg_slot = seg_slot;
  a.heads = heads; a.dk = n_state; a.dv = dv;
  a.state = state; a.state_slot_stride = prl_lin_scan_state_floats(heads, n_state, dv);
  a.out = out; a.ld_out = ld_out;
  a.kvec = xbc; a.ld_k = ld_xbc; a.off_k = inner;                         // B: [groups][state] after x
  a.qvec = xbc; a.ld_q = ld_xbc; a.off_q = inner + groups * n_state;      // C
  a.xval = xbc; a.ld_x = ld_xbc; a.off_x = 0;
  a.q_scale = 1.f;
  a.dt_raw = P; a.ld_dt = ldp; a.off_dt = off_dt; a.groups = groups;
  a.dt_bias = dt_bias; a.a_log = a_log; a.skip = skip;
  if (split) return launch_split<kSsd>(a, n_seg, *split, n_sub, (cudaStream_t)st);
  return launch_scan<kSsd>(a, n_seg, (cudaStream_t)st);
}

extern "C" int prl_ssd_scan(const float* P, int64_t ldp, int32_t off_dt, const float* xbc, int64_t ld_xbc,
                            const float* dt_bias, const float* a_log, const float* skip, int32_t heads, int32_t groups,
                            int32_t n_state, int32_t dv, const int32_t* seg_start, const int32_t* seg_len,
                            const int32_t* seg_slot, int32_t n_seg, float* state, float* out, int64_t ld_out,
                            prl_stream_t st) {
  return ssd_scan_impl(P, ldp, off_dt, xbc, ld_xbc, dt_bias, a_log, skip, heads, groups, n_state, dv, seg_start, seg_len,
                       seg_slot, n_seg, state, out, ld_out, nullptr, 0, st);
}

extern "C" int prl_ssd_scan_split(const float* P, int64_t ldp, int32_t off_dt, const float* xbc, int64_t ld_xbc,
                                  const float* dt_bias, const float* a_log, const float* skip, int32_t heads, int32_t groups,
                                  int32_t n_state, int32_t dv, const int32_t* seg_slot, int32_t n_seg,
                                  const int32_t* seg_sub0, const int32_t* seg_nsub, const int32_t* sub_start,
                                  const int32_t* sub_len, int32_t n_sub, float* scratch, float* cdec, float* state,
                                  float* out, int64_t ld_out, prl_stream_t st) {
  SplitArgs p;
  PRL_CHECK_ARG(split_args(p, seg_sub0, seg_nsub, sub_start, sub_len, n_sub, scratch, cdec), "prl_ssd_scan_split: bad piece tables");
  return ssd_scan_impl(P, ldp, off_dt, xbc, ld_xbc, dt_bias, a_log, skip, heads, groups, n_state, dv, sub_start, sub_len,
                       seg_slot, n_seg, state, out, ld_out, &p, n_sub, st);
}

// ---- SCALAR front end: S_t = a_t S_(t-1) + b_t k_t v_t^T, o_t = q_scale * S_t^T q_t ----------------------------------
// q, k: columns off_q / off_k (+ head * dk) of P; values: columns off_x (+ head * dv) of `xval` (which may be P).
// gates != NULL: (a_t, b_t) = gates[row * ld_g + off_g + 2 * head + {0, 1}]; otherwise a_t = const_decay[head], b_t = 1.
static int decay_scan_impl(const float* P, int64_t ldp, int32_t off_q, int32_t off_k, float q_scale, const float* xval,
                           int64_t ld_x, int32_t off_x, const float* gates, int64_t ld_g, int32_t off_g,
                           const float* const_decay, int32_t heads, int32_t dk, int32_t dv, const int32_t* seg_start,
                           const int32_t* seg_len, const int32_t* seg_slot, int32_t n_seg, float* state, float* out,
                           int64_t ld_out, const SplitArgs* split, int32_t n_sub, prl_stream_t st) {
  PRL_CHECK_ARG(P && xval && (gates || const_decay) && seg_start && seg_len && seg_slot && state && out,
                "prl_decay_scan: NULL argument");
  PRL_CHECK_ARG(heads >= 1 && dk >= 1 && dk <= 256 && dv >= 1 && n_seg >= 1 && n_seg <= 65535,
                "prl_decay_scan: bad shape (heads=%d dk=%d dv=%d, dk at most 256)", heads, dk, dv);
  ScanArgs a = {};
  a.seg_start = seg_start; a.seg_len = seg_len; a.seg_slot = seg_slot;
  a.heads = heads; a.dk = dk; a.dv = dv;
  a.state = state; a.state_slot_stride = prl_lin_scan_state_floats(heads, dk, dv);
  a.out = out; a.ld_out = ld_out;
  a.kvec = P; a.ld_k = ldp; a.off_k = off_k;
  a.qvec = P; a.ld_q = ldp; a.off_q = off_q;
  a.xval = xval; a.ld_x = ld_x; a.off_x = off_x;
  a.q_scale = q_scale;
  a.dt_raw = gates; a.ld_dt = ld_g; a.off_dt = off_g; a.groups = heads;
  a.a_log = const_decay;
  if (split) return launch_split<kScalar>(a, n_seg, *split, n_sub, (cudaStream_t)st);
  return launch_scan<kScalar>(a, n_seg, (cudaStream_t)st);
}

extern "C" int prl_decay_scan(const float* P, int64_t ldp, int32_t off_q, int32_t off_k, float q_scale, const float* xval,
                              int64_t ld_x, int32_t off_x, const float* gates, int64_t ld_g, int32_t off_g,
                              const float* const_decay, int32_t heads, int32_t dk, int32_t dv, const int32_t* seg_start,
                              const int32_t* seg_len, const int32_t* seg_slot, int32_t n_seg, float* state, float* out,
                              int64_t ld_out, prl_stream_t st) {
  return decay_scan_impl(P, ldp, off_q, off_k, q_scale, xval, ld_x, off_x, gates, ld_g, off_g, const_decay, heads, dk, dv,
                         seg_start, seg_len, seg_slot, n_seg, state, out, ld_out, nullptr, 0, st);
}

// The same with every segment cut into side-by-side pieces (see prl_gla_scan_split for the tables).
extern "C" int prl_decay_scan_split(const float* P, int64_t ldp, int32_t off_q, int32_t off_k, float q_scale,
                                    const float* xval, int64_t ld_x, int32_t off_x, const float* gates, int64_t ld_g,
                                    int32_t off_g, const float* const_decay, int32_t heads, int32_t dk, int32_t dv,
                                    const int32_t* seg_slot, int32_t n_seg, const int32_t* seg_sub0,
                                    const int32_t* seg_nsub, const int32_t* sub_start, const int32_t* sub_len,
                                    int32_t n_sub, float* scratch, float* cdec, float* state, float* out, int64_t ld_out,
                                    prl_stream_t st) {
  SplitArgs p;
  PRL_CHECK_ARG(split_args(p, seg_sub0, seg_nsub, sub_start, sub_len, n_sub, scratch, cdec), "prl_decay_scan_split: bad piece tables");
  return decay_scan_impl(P, ldp, off_q, off_k, q_scale, xval, ld_x, off_x, gates, ld_g, off_g, const_decay, heads, dk, dv,
                         sub_start, sub_len, seg_slot, n_seg, state, out, ld_out, &p, n_sub, st);
}
