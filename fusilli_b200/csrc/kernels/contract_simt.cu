// CUDA-core implicit-GEMM kernel for every contraction the tensor-core kernels do
// not take: fp32 operands (which need fp32-accurate products), grouped / strided /
// dilated / 1-D / 3-D / NCHW convolutions, odd extents, transposed or broadcast
// matmul operands. One kernel, four index mappings:
//
//   matmul  C[g][m][n]  = sum_k A[g][m][k] * B[g][k][n]
//   fprop   Y[n,ko,o..] = sum_{c,taps} X[n,c,o*s-p+tap*d] * W[ko,c,taps]
//   dgrad   DX[n,c,i..] = sum_{ko,taps} DY[n,ko,(i+p-tap*d)/s] * W[ko,c,taps]
//   wgrad   DW[ko,c,taps] = sum_{n,o..} DY[n,ko,o..] * X[n,c,o*s-p+tap*d]
//
// 64x64x16 tiles, 256 threads, 4x4 register micro-tile, fp32 FFMA accumulation,
// operands converted to fp32 while staging into shared memory, trailing pointwise
// nodes applied in the epilogue. wgrad splits its long reduction across CTAs:
// fp32 partial tiles go to the workspace and a second kernel sums them in a fixed
// order (deterministic) before the epilogue.
#include "../common.h"

namespace fb {

enum { CM_MATMUL = 0, CM_FPROP = 1, CM_DGRAD = 2, CM_WGRAD = 3 };

struct ConvGeomDev {
  int32_t N, C, D, H, W, K, Cg, Kg, T, R, S, OD, OH, OW;
  int32_t pd, ph, pw, sd, sh, sw, dd, dh, dw;
  int32_t nsp;
  int32_t chan_fastest; // reduction index ordered (taps, channel) instead of (channel, taps)
  int64_t xs[5], ws[5], ys[5]; // element strides of x-like, w-like, y-like tensors (n,c,d,h,w)
};

struct ContractParams {
  int32_t mode;
  int32_t a_dtype, b_dtype;
  int32_t a_kfast, b_nfast;
  int32_t G, split_k;
  const void *a, *b;
  void *out;
  float *partial;
  int64_t M, N, K, k_chunk;
  // matmul addressing
  int32_t nbatch_dims;
  int64_t bdims[6], a_bdims[6], b_bdims[6], a_bstr[6], b_bstr[6], c_bstr[6];
  int64_t a_sm, a_sk, b_sk, b_sn, c_sm, c_sn;
  ConvGeomDev g;
  EpilogueDev epi;
};

constexpr int BM = 64, BN = 64, BK = 16;

__device__ __forceinline__ void batch_offsets(const ContractParams &p, int g, int64_t &ao, int64_t &bo,
                                              int64_t &co, int64_t *idx) {
  ao = bo = co = 0;
  int rem = g;
  for (int d = p.nbatch_dims - 1; d >= 0; --d) {
    int c = rem % (int)p.bdims[d];
    rem /= (int)p.bdims[d];
    // an operand whose batch dim divides the result's is read modulo (reference
    // matmul_node.h:140-150 accepts such dims; 1 is the usual broadcast)
    ao += (c % (int)p.a_bdims[d]) * p.a_bstr[d];
    bo += (c % (int)p.b_bdims[d]) * p.b_bstr[d];
    co += c * p.c_bstr[d];
    if (idx) idx[d] = c;
  }
}

// Reduction index -> (channel-in-group, t, r, s)
__device__ __forceinline__ void split_taps(const ConvGeomDev &g, int k, int nchan, int &ch, int &t, int &r, int &s) {
  if (g.chan_fastest) {
    ch = k % nchan; k /= nchan;
    s = k % g.S; k /= g.S;
    r = k % g.R; k /= g.R;
    t = k;
  } else {
    s = k % g.S; k /= g.S;
    r = k % g.R; k /= g.R;
    t = k % g.T; k /= g.T;
    ch = k;
  }
}

__device__ __forceinline__ void split_pos(int m, int d1, int d2, int d3, int &n, int &a, int &b, int &c) {
  c = m % d3; m /= d3;
  b = m % d2; m /= d2;
  a = m % d1; m /= d1;
  n = m;
}

// A(g, m, k) as fp32, 0 outside the problem or in the padding halo.
__device__ __forceinline__ float fetch_a(const ContractParams &p, int g, int64_t abase, int m, int k) {
  if (m >= p.M || k >= p.K) return 0.f;
  const ConvGeomDev &q = p.g;
  switch (p.mode) {
  case CM_MATMUL: return load_f(p.a, p.a_dtype, abase + (int64_t)m * p.a_sm + (int64_t)k * p.a_sk);
  case CM_FPROP: {
    int n, od, oh, ow, cg, t, r, s;
    split_pos(m, q.OD, q.OH, q.OW, n, od, oh, ow);
    split_taps(q, k, q.Cg, cg, t, r, s);
    int id = od * q.sd - q.pd + t * q.dd, ih = oh * q.sh - q.ph + r * q.dh, iw = ow * q.sw - q.pw + s * q.dw;
    if (id < 0 || id >= q.D || ih < 0 || ih >= q.H || iw < 0 || iw >= q.W) return 0.f;
    int c = g * q.Cg + cg;
    return load_f(p.a, p.a_dtype, n * q.xs[0] + c * q.xs[1] + id * q.xs[2] + ih * q.xs[3] + iw * q.xs[4]);
  }
  case CM_DGRAD: {
    int n, id, ih, iw, kk, t, r, s;
    split_pos(m, q.D, q.H, q.W, n, id, ih, iw);
    split_taps(q, k, q.Kg, kk, t, r, s);
    int nd = id + q.pd - t * q.dd, nh = ih + q.ph - r * q.dh, nw = iw + q.pw - s * q.dw;
    if (nd < 0 || nh < 0 || nw < 0) return 0.f;
    if (nd % q.sd || nh % q.sh || nw % q.sw) return 0.f;
    int od = nd / q.sd, oh = nh / q.sh, ow = nw / q.sw;
    if (od >= q.OD || oh >= q.OH || ow >= q.OW) return 0.f;
    int ko = g * q.Kg + kk;
    return load_f(p.a, p.a_dtype, n * q.ys[0] + ko * q.ys[1] + od * q.ys[2] + oh * q.ys[3] + ow * q.ys[4]);
  }
  default: { // CM_WGRAD: A = DY[n, ko, o..]
    int n, od, oh, ow;
    split_pos(k, q.OD, q.OH, q.OW, n, od, oh, ow);
    int ko = g * q.Kg + m;
    return load_f(p.a, p.a_dtype, n * q.ys[0] + ko * q.ys[1] + od * q.ys[2] + oh * q.ys[3] + ow * q.ys[4]);
  }
  }
}

__device__ __forceinline__ float fetch_b(const ContractParams &p, int g, int64_t bbase, int k, int nn) {
  if (nn >= p.N || k >= p.K) return 0.f;
  const ConvGeomDev &q = p.g;
  switch (p.mode) {
  case CM_MATMUL: return load_f(p.b, p.b_dtype, bbase + (int64_t)k * p.b_sk + (int64_t)nn * p.b_sn);
  case CM_FPROP: {
    int cg, t, r, s;
    split_taps(q, k, q.Cg, cg, t, r, s);
    int ko = g * q.Kg + nn;
    return load_f(p.b, p.b_dtype, ko * q.ws[0] + cg * q.ws[1] + t * q.ws[2] + r * q.ws[3] + s * q.ws[4]);
  }
  case CM_DGRAD: {
    int kk, t, r, s;
    split_taps(q, k, q.Kg, kk, t, r, s);
    int ko = g * q.Kg + kk;
    return load_f(p.b, p.b_dtype, ko * q.ws[0] + nn * q.ws[1] + t * q.ws[2] + r * q.ws[3] + s * q.ws[4]);
  }
  default: { // CM_WGRAD: B = X[n, c, o*s-p+tap*d], column nn = (cg, taps)
    int n, od, oh, ow, cg, t, r, s;
    split_pos(k, q.OD, q.OH, q.OW, n, od, oh, ow);
    split_taps(q, nn, q.Cg, cg, t, r, s);
    int id = od * q.sd - q.pd + t * q.dd, ih = oh * q.sh - q.ph + r * q.dh, iw = ow * q.sw - q.pw + s * q.dw;
    if (id < 0 || id >= q.D || ih < 0 || ih >= q.H || iw < 0 || iw >= q.W) return 0.f;
    int c = g * q.Cg + cg;
    return load_f(p.b, p.b_dtype, n * q.xs[0] + c * q.xs[1] + id * q.xs[2] + ih * q.xs[3] + iw * q.xs[4]);
  }
  }
}

// Epilogue + store of output element (g, m, nn).
__device__ __forceinline__ void store_out(const ContractParams &p, int g, int m, int nn, float acc) {
  const ConvGeomDev &q = p.g;
  int64_t idx[FB_MAX_RANK];
  int64_t off;
  switch (p.mode) {
  case CM_MATMUL: {
    int64_t ao, bo, co;
    batch_offsets(p, g, ao, bo, co, idx);
    idx[p.nbatch_dims] = m;
    idx[p.nbatch_dims + 1] = nn;
    off = co + (int64_t)m * p.c_sm + (int64_t)nn * p.c_sn;
  } break;
  case CM_FPROP: {
    int n, od, oh, ow;
    split_pos(m, q.OD, q.OH, q.OW, n, od, oh, ow);
    int ko = g * q.Kg + nn;
    idx[0] = n; idx[1] = ko;
    int sp[3] = {od, oh, ow};
    for (int i = 0; i < q.nsp; ++i) idx[2 + i] = sp[3 - q.nsp + i];
    off = n * q.ys[0] + ko * q.ys[1] + od * q.ys[2] + oh * q.ys[3] + ow * q.ys[4];
  } break;
  case CM_DGRAD: {
    int n, id, ih, iw;
    split_pos(m, q.D, q.H, q.W, n, id, ih, iw);
    int c = g * q.Cg + nn;
    idx[0] = n; idx[1] = c;
    int sp[3] = {id, ih, iw};
    for (int i = 0; i < q.nsp; ++i) idx[2 + i] = sp[3 - q.nsp + i];
    off = n * q.xs[0] + c * q.xs[1] + id * q.xs[2] + ih * q.xs[3] + iw * q.xs[4];
  } break;
  default: {
    int cg, t, r, s;
    split_taps(q, nn, q.Cg, cg, t, r, s);
    int ko = g * q.Kg + m;
    idx[0] = ko; idx[1] = cg;
    int sp[3] = {t, r, s};
    for (int i = 0; i < q.nsp; ++i) idx[2 + i] = sp[3 - q.nsp + i];
    off = ko * q.ws[0] + cg * q.ws[1] + t * q.ws[2] + r * q.ws[3] + s * q.ws[4];
  } break;
  }
  store_f(p.out, p.epi.out_dtype, off, apply_epilogue(p.epi, acc, idx));
}

__global__ void __launch_bounds__(256) contract_simt_kernel(const ContractParams p) {
  __shared__ __align__(16) float As[BK][BM + 4];
  __shared__ __align__(16) float Bs[BK][BN + 4];
  const int tid = threadIdx.x;
  const int g = blockIdx.z / p.split_k, sp = blockIdx.z % p.split_k;
  const int m0 = blockIdx.x * BM, n0 = blockIdx.y * BN;
  int64_t abase = 0, bbase = 0, cbase = 0;
  if (p.mode == CM_MATMUL) batch_offsets(p, g, abase, bbase, cbase, nullptr);
  const int k_begin = (int)(sp * p.k_chunk);
  const int k_end = (int)min((int64_t)p.K, (int64_t)(sp + 1) * p.k_chunk);
  // staging assignment: 4 A elements and 4 B elements per thread per k-tile
  int a_m[4], a_k[4], b_k[4], b_n[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    if (p.a_kfast) { a_k[i] = tid % BK; a_m[i] = tid / BK + 16 * i; }
    else           { a_m[i] = tid % BM; a_k[i] = tid / BM + 4 * i; }
    if (p.b_nfast) { b_n[i] = tid % BN; b_k[i] = tid / BN + 4 * i; }
    else           { b_k[i] = tid % BK; b_n[i] = tid / BK + 16 * i; }
  }
  const int tx = tid % 16, ty = tid / 16;
  float acc[4][4] = {};
  float ra[4], rb[4];
  auto fetch_tile = [&](int k0) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      int ka = k0 + a_k[i], kb = k0 + b_k[i];
      ra[i] = (ka < k_end) ? fetch_a(p, g, abase, m0 + a_m[i], ka) : 0.f;
      rb[i] = (kb < k_end) ? fetch_b(p, g, bbase, kb, n0 + b_n[i]) : 0.f;
    }
  };
  if (k_begin < k_end) fetch_tile(k_begin);
  for (int k0 = k_begin; k0 < k_end; k0 += BK) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      As[a_k[i]][a_m[i]] = ra[i];
      Bs[b_k[i]][b_n[i]] = rb[i];
    }
    __syncthreads();
    if (k0 + BK < k_end) fetch_tile(k0 + BK);
#pragma unroll
    for (int kk = 0; kk < BK; ++kk) {
      float4 av = *reinterpret_cast<const float4 *>(&As[kk][ty * 4]);
      float4 bv = *reinterpret_cast<const float4 *>(&Bs[kk][tx * 4]);
      float a4[4] = {av.x, av.y, av.z, av.w}, b4[4] = {bv.x, bv.y, bv.z, bv.w};
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a4[i], b4[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    int m = m0 + ty * 4 + i;
    if (m >= p.M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      int nn = n0 + tx * 4 + j;
      if (nn >= p.N) continue;
      if (p.split_k > 1)
        p.partial[(((int64_t)sp * p.G + g) * p.M + m) * p.N + nn] = acc[i][j];
      else
        store_out(p, g, m, nn, acc[i][j]);
    }
  }
}

// Channels-last fp32 forward convolution (2-D, channel count a multiple of 16): the same implicit
// GEMM as above with the index arithmetic hoisted out of the loop. A 16-wide reduction tile is 16
// consecutive channels of ONE filter tap, so per tile a thread does one bounds test and one
// 16-byte load per pixel row instead of a full coordinate decomposition per element. Tile 128
// pixels x 64 output channels x 16, 8 x 4 outputs per thread, next tile prefetched in registers.
constexpr int FBM = 128, FBN = 64, FBK = 16;
__global__ void __launch_bounds__(256, 3) conv_fprop_cl_f32_kernel(const ContractParams p) {
  __shared__ __align__(16) float As[FBK][FBM + 4];
  __shared__ __align__(16) float Bs[FBK][FBN + 4];
  const ConvGeomDev &q = p.g;
  const int tid = threadIdx.x;
  const int g = blockIdx.z;
  const int m0 = blockIdx.x * FBM, n0 = blockIdx.y * FBN;
  const float *x = static_cast<const float *>(p.a), *wt = static_cast<const float *>(p.b);
  // staging: two pixel rows and one filter row per thread, four consecutive channels each
  const int k4 = (tid & 3) * 4;
  const float *a_img[2]; // image base of the row's pixel (channel group applied)
  int a_ih0[2], a_iw0[2];
  bool a_ok[2];
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int m = m0 + (tid >> 2) + 64 * i;
    a_ok[i] = m < p.M;
    int n, od, oh, ow;
    split_pos(a_ok[i] ? m : 0, q.OD, q.OH, q.OW, n, od, oh, ow);
    a_img[i] = x + (int64_t)n * q.xs[0] + (int64_t)g * q.Cg + k4;
    a_ih0[i] = oh * q.sh - q.ph;
    a_iw0[i] = ow * q.sw - q.pw;
  }
  const int b_n = n0 + (tid >> 2);
  const bool b_ok = b_n < p.N;
  const float *b_row = wt + (int64_t)(g * q.Kg + (b_ok ? b_n : 0)) * q.ws[0] + k4;
  const int tx = tid & 15, ty = tid >> 4; // outputs: rows ty*8 .. +7, columns tx*4 .. +3
  float acc[8][4] = {};
  float4 ra[2], rb;
  // The reduction walks (filter row, filter column, 16-channel block) with counters: per tap one
  // bounds test and one pointer per staged row, per block one 16-byte load per row.
  int tr = 0, ts = 0, c0 = 0;
  const float *a_tap[2], *b_tap;
  auto enter_tap = [&]() {
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int ih = a_ih0[i] + tr * q.dh, iw = a_iw0[i] + ts * q.dw;
      const bool in = a_ok[i] && ih >= 0 && ih < q.H && iw >= 0 && iw < q.W;
      a_tap[i] = in ? a_img[i] + (int64_t)ih * q.xs[3] + (int64_t)iw * q.xs[4] : nullptr;
    }
    b_tap = b_ok ? b_row + (int64_t)tr * q.ws[3] + (int64_t)ts * q.ws[4] : nullptr;
  };
  auto fetch_tile = [&]() {
#pragma unroll
    for (int i = 0; i < 2; ++i)
      ra[i] = a_tap[i] ? __ldg(reinterpret_cast<const float4 *>(a_tap[i] + c0)) : make_float4(0.f, 0.f, 0.f, 0.f);
    rb = b_tap ? __ldg(reinterpret_cast<const float4 *>(b_tap + c0)) : make_float4(0.f, 0.f, 0.f, 0.f);
    c0 += FBK;
    if (c0 == q.Cg) {
      c0 = 0;
      if (++ts == q.S) {
        ts = 0;
        ++tr;
      }
      enter_tap();
    }
  };
  const int K = (int)p.K;
  enter_tap();
  fetch_tile();
  for (int k0 = 0; k0 < K; k0 += FBK) {
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int m = (tid >> 2) + 64 * i;
      As[k4 + 0][m] = ra[i].x; As[k4 + 1][m] = ra[i].y; As[k4 + 2][m] = ra[i].z; As[k4 + 3][m] = ra[i].w;
    }
    Bs[k4 + 0][tid >> 2] = rb.x; Bs[k4 + 1][tid >> 2] = rb.y; Bs[k4 + 2][tid >> 2] = rb.z; Bs[k4 + 3][tid >> 2] = rb.w;
    __syncthreads();
    if (k0 + FBK < K) fetch_tile();
#pragma unroll
    for (int kk = 0; kk < FBK; ++kk) {
      const float4 a0 = *reinterpret_cast<const float4 *>(&As[kk][ty * 8]);
      const float4 a1 = *reinterpret_cast<const float4 *>(&As[kk][ty * 8 + 4]);
      const float4 bv = *reinterpret_cast<const float4 *>(&Bs[kk][tx * 4]);
      const float a8[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w}, b4[4] = {bv.x, bv.y, bv.z, bv.w};
#pragma unroll
      for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a8[i], b4[j], acc[i][j]);
    }
    __syncthreads();
  }
  // Epilogue: the pixel decomposition and every operand's offset are taken once per output row;
  // the four channels of a row differ only in the channel term.
  const EpilogueDev &e = p.epi;
  const int ko0 = g * q.Kg + n0 + tx * 4;
  const bool row_vec = e.out_dtype == FB_DT_FLOAT && q.ys[1] == 1 && n0 + tx * 4 + 3 < p.N &&
                       (reinterpret_cast<uintptr_t>(p.out) & 15) == 0 && (ko0 & 3) == 0;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int m = m0 + ty * 8 + i;
    if (m >= p.M) break;
    int n, od, oh, ow;
    split_pos(m, q.OD, q.OH, q.OW, n, od, oh, ow);
    const int sp[3] = {od, oh, ow};
    const int64_t out_row = n * q.ys[0] + od * q.ys[2] + oh * q.ys[3] + ow * q.ys[4];
    int64_t op_row[kMaxEpiOps], op_cs[kMaxEpiOps];
#pragma unroll
    for (int o = 0; o < kMaxEpiOps; ++o) {
      op_row[o] = 0;
      op_cs[o] = 0;
      if (o < e.num_ops && e.ops[o].operand_kind == 1) {
        int64_t off = n * e.ops[o].strides[0];
        for (int d = 0; d < q.nsp; ++d) off += sp[3 - q.nsp + d] * e.ops[o].strides[2 + d];
        op_row[o] = off;
        op_cs[o] = e.ops[o].strides[1];
      }
    }
    float v[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int ko = ko0 + j;
      float r = round_to(acc[i][j], e.acc_round_dtype);
#pragma unroll
      for (int o = 0; o < kMaxEpiOps; ++o) {
        if (o >= e.num_ops) break;
        const EpiOpDev &op = e.ops[o];
        float other = 0.f;
        if (op.operand_kind == 1) other = load_f(op.operand, op.operand_dtype, op_row[o] + ko * op_cs[o]);
        else if (op.operand_kind == 2) other = op.scalar;
        const float a = op.value_is_in1 ? other : r, b = op.value_is_in1 ? r : other;
        r = round_to(pw_apply_f(op.mode, a, b, 0.f, op.fparams), op.round_dtype);
      }
      v[j] = r;
    }
    if (row_vec) {
      *reinterpret_cast<float4 *>(static_cast<float *>(p.out) + out_row + ko0) = make_float4(v[0], v[1], v[2], v[3]);
    } else {
#pragma unroll
      for (int j = 0; j < 4; ++j)
        if (n0 + tx * 4 + j < p.N) store_f(p.out, e.out_dtype, out_row + (int64_t)(ko0 + j) * q.ys[1], v[j]);
    }
  }
}

// Sums the split-K partial tiles in split order, then epilogue + store.
__global__ void __launch_bounds__(256) contract_splitk_reduce_kernel(const ContractParams p) {
  int64_t total = (int64_t)p.G * p.M * p.N;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (int64_t)gridDim.x * blockDim.x) {
    float acc = 0.f;
    for (int s = 0; s < p.split_k; ++s) acc += p.partial[(int64_t)s * total + i];
    int nn = (int)(i % p.N);
    int64_t rest = i / p.N;
    int m = (int)(rest % p.M);
    int g = (int)(rest / p.M);
    store_out(p, g, m, nn, acc);
  }
}

static void fill_strides5(const TensorInfo &t, int nsp, int64_t *out) {
  out[0] = t.strides[0];
  out[1] = t.strides[1];
  for (int i = 0; i < 3; ++i) out[2 + i] = 0;
  for (int i = 0; i < nsp; ++i) out[2 + (3 - nsp) + i] = t.strides[2 + i];
}

static void fill_dims5(const TensorInfo &t, int nsp, int32_t *n, int32_t *c, int32_t *d, int32_t *h, int32_t *w) {
  int32_t sp[3] = {1, 1, 1};
  for (int i = 0; i < nsp; ++i) sp[3 - nsp + i] = (int32_t)t.dims[2 + i];
  *n = (int32_t)t.dims[0];
  *c = (int32_t)t.dims[1];
  *d = sp[0]; *h = sp[1]; *w = sp[2];
}

fb_status launch_contract_simt(const ExecContext &cx, const Step &s) {
  const Plan &plan = *cx.plan;
  const fb_node_desc &d = plan.nodes[s.node].d;
  static thread_local ContractParams p; // large POD; avoid re-zeroing the stack each call
  memset(&p, 0, sizeof(p));
  fb_status st = build_epilogue(cx, s, p.epi);
  if (st != FB_OK) return st;
  const TensorInfo &t0 = plan.tensors[d.inputs[0]], &t1 = plan.tensors[d.inputs[1]];
  const TensorInfo &to = plan.tensors[d.outputs[0]];
  p.a = cx.tensor_ptr(d.inputs[0]);
  p.b = cx.tensor_ptr(d.inputs[1]);
  p.out = cx.tensor_ptr(s.out_tensor);
  FB_REQUIRE(p.a && p.b && p.out, FB_INTERNAL_ERROR, "contract: tensor has no buffer");
  p.a_dtype = t0.dtype;
  p.b_dtype = t1.dtype;
  p.split_k = 1;
  if (d.op == FB_OP_MATMUL) {
    p.mode = CM_MATMUL;
    int r = t0.rank;
    p.M = t0.dims[r - 2];
    p.K = t0.dims[r - 1];
    p.N = t1.dims[r - 1];
    p.a_sm = t0.strides[r - 2]; p.a_sk = t0.strides[r - 1];
    p.b_sk = t1.strides[r - 2]; p.b_sn = t1.strides[r - 1];
    // the stored tensor may be a later pointwise output with its own strides
    const TensorInfo &tc = plan.tensors[s.out_tensor];
    p.c_sm = tc.strides[r - 2]; p.c_sn = tc.strides[r - 1];
    p.nbatch_dims = r - 2;
    FB_REQUIRE(p.nbatch_dims <= 6, FB_NOT_IMPLEMENTED, "matmul: more than 6 batch dims");
    int64_t G = 1;
    for (int i = 0; i < r - 2; ++i) {
      p.bdims[i] = to.dims[i];
      p.a_bstr[i] = t0.dims[i] == 1 ? 0 : t0.strides[i];
      p.b_bstr[i] = t1.dims[i] == 1 ? 0 : t1.strides[i];
      p.a_bdims[i] = t0.dims[i];
      p.b_bdims[i] = t1.dims[i];
      FB_REQUIRE(to.dims[i] % t0.dims[i] == 0 && to.dims[i] % t1.dims[i] == 0, FB_INVALID_ARGUMENT,
                 "matmul: a batch dim of an operand does not divide the result's");
      p.c_bstr[i] = tc.strides[i];
      G *= to.dims[i];
    }
    p.G = (int32_t)G;
    p.a_kfast = (p.a_sk == 1) ? 1 : 0;
    p.b_nfast = (p.b_sn == 1) ? 1 : 0;
  } else {
    ConvGeomDev &g = p.g;
    g.nsp = d.num_spatial;
    const TensorInfo *tx, *tw, *ty;
    if (d.op == FB_OP_CONV_FPROP) { p.mode = CM_FPROP; tx = &t0; tw = &t1; ty = &to; }
    else if (d.op == FB_OP_CONV_DGRAD) { p.mode = CM_DGRAD; ty = &t0; tw = &t1; tx = &to; }
    else { p.mode = CM_WGRAD; ty = &t0; tx = &t1; tw = &to; }
    // the tensor actually written may be a later pointwise output (same dims)
    const TensorInfo &tst = plan.tensors[s.out_tensor];
    fill_dims5(*tx, g.nsp, &g.N, &g.C, &g.D, &g.H, &g.W);
    int32_t dummy;
    fill_dims5(*tw, g.nsp, &g.K, &g.Cg, &g.T, &g.R, &g.S);
    fill_dims5(*ty, g.nsp, &dummy, &dummy, &g.OD, &g.OH, &g.OW);
    fill_strides5(p.mode == CM_DGRAD ? tst : *tx, g.nsp, g.xs);
    fill_strides5(p.mode == CM_WGRAD ? tst : *tw, g.nsp, g.ws);
    fill_strides5(p.mode == CM_FPROP ? tst : *ty, g.nsp, g.ys);
    int32_t pad[3] = {0, 0, 0}, str[3] = {1, 1, 1}, dil[3] = {1, 1, 1};
    for (int i = 0; i < g.nsp; ++i) {
      pad[3 - g.nsp + i] = (int32_t)d.padding[i];
      str[3 - g.nsp + i] = (int32_t)d.stride[i];
      dil[3 - g.nsp + i] = (int32_t)d.dilation[i];
    }
    g.pd = pad[0]; g.ph = pad[1]; g.pw = pad[2];
    g.sd = str[0]; g.sh = str[1]; g.sw = str[2];
    g.dd = dil[0]; g.dh = dil[1]; g.dw = dil[2];
    int groups = g.C / g.Cg;
    g.Kg = g.K / groups;
    p.G = groups;
    bool x_cl = tx->strides[1] == 1 && tx->dims[1] > 1;
    bool w_cl = tw->strides[1] == 1 && tw->dims[1] > 1;
    bool y_cl = ty->strides[1] == 1 && ty->dims[1] > 1;
    int64_t npos_out = (int64_t)g.N * g.OD * g.OH * g.OW, npos_in = (int64_t)g.N * g.D * g.H * g.W;
    int64_t taps = (int64_t)g.T * g.R * g.S;
    if (p.mode == CM_FPROP) {
      p.M = npos_out; p.N = g.Kg; p.K = g.Cg * taps;
      g.chan_fastest = x_cl && w_cl;
      p.a_kfast = x_cl ? 1 : 0;
      p.b_nfast = 0;
    } else if (p.mode == CM_DGRAD) {
      p.M = npos_in; p.N = g.Cg; p.K = g.Kg * taps;
      g.chan_fastest = y_cl;
      p.a_kfast = y_cl ? 1 : 0;
      p.b_nfast = w_cl ? 1 : 0;
    } else {
      p.M = g.Kg; p.N = g.Cg * taps; p.K = npos_out;
      g.chan_fastest = x_cl;
      p.a_kfast = y_cl ? 0 : 1;
      p.b_nfast = x_cl ? 1 : 0;
      p.split_k = s.split_k;
    }
    FB_REQUIRE(p.M < (1ll << 31) && p.K < (1ll << 31) && p.N < (1ll << 31), FB_NOT_IMPLEMENTED,
               "conv: problem extent exceeds 2^31");
  }
  p.k_chunk = ((p.K + p.split_k - 1) / p.split_k + BK - 1) / BK * BK;
  if (p.split_k > 1) {
    FB_REQUIRE(cx.workspace && s.scratch_offset >= 0, FB_INTERNAL_ERROR, "wgrad: split-K scratch missing");
    p.partial = reinterpret_cast<float *>(cx.workspace + s.scratch_offset);
  }
  dim3 grid((unsigned)((p.M + BM - 1) / BM), (unsigned)((p.N + BN - 1) / BN), (unsigned)(p.G * p.split_k));
  if (grid.y > 65535 || grid.z > 65535)
    return fail(FB_NOT_IMPLEMENTED, "contract: problem too large for the CUDA-core kernel's grid");
  cudaStream_t stream = cx.dev->stream;
  if (p.mode == CM_FPROP && p.g.chan_fastest && p.a_dtype == FB_DT_FLOAT && p.b_dtype == FB_DT_FLOAT &&
      p.g.nsp == 2 && p.g.Cg % FBK == 0 && p.g.xs[1] == 1 && p.g.ws[1] == 1 &&
      (reinterpret_cast<uintptr_t>(p.a) & 15) == 0 && (reinterpret_cast<uintptr_t>(p.b) & 15) == 0 &&
      p.g.xs[0] % 4 == 0 && p.g.xs[3] % 4 == 0 && p.g.xs[4] % 4 == 0 && p.g.ws[0] % 4 == 0 && p.g.ws[3] % 4 == 0 &&
      p.g.ws[4] % 4 == 0) {
    dim3 fgrid((unsigned)((p.M + FBM - 1) / FBM), (unsigned)((p.N + FBN - 1) / FBN), (unsigned)p.G);
    if (fgrid.y <= 65535 && fgrid.z <= 65535) {
      conv_fprop_cl_f32_kernel<<<fgrid, 256, 0, stream>>>(p);
      return FB_OK;
    }
  }
  contract_simt_kernel<<<grid, 256, 0, stream>>>(p);
  if (p.split_k > 1) {
    int64_t total = (int64_t)p.G * p.M * p.N;
    int blocks = (int)std::min<int64_t>((total + 255) / 256, (int64_t)cx.dev->sm_count * 8);
    contract_splitk_reduce_kernel<<<blocks, 256, 0, stream>>>(p);
  }
  return FB_OK;
}

} // namespace fb

// ---------------------------------------------------------------------------------
// Allocation-free weight-gradient entry point.
//
// fb_plan_execute takes its split-K scratch from a caller-provided workspace, which
// somebody had to allocate. Some callers cannot allocate at all at the point where
// they need the result: code running inside a framework's allocator callback or
// under its allocator lock, a real-time loop with a no-allocation rule, a plugin
// that is handed raw device pointers and a stream and nothing else. For them this
// entry point keeps the scratch in a fixed array inside the library image.
//
// The array lives in device memory of every GPU that loads the library, for the
// life of the process. In host code the name `g_wgrad_static_scratch` is only a
// handle for the symbol, not a device address, so its address is resolved once per
// device with cudaGetSymbolAddress and that pointer is what the kernels receive.
// ---------------------------------------------------------------------------------

#include <mutex>

namespace fb {
namespace {

constexpr size_t kStaticScratchBytes = 8u << 20; // 8 MiB per GPU
__device__ __align__(256) float g_wgrad_static_scratch[kStaticScratchBytes / sizeof(float)];

constexpr int kMaxDevices = 64;
std::mutex g_static_scratch_mutex;
float *g_static_scratch_ptr[kMaxDevices] = {nullptr};
int g_static_sm_count[kMaxDevices] = {0};

// Device address of the scratch array on the CURRENT device and that device's SM count, both
// resolved on the first call per device. That first call may make the CUDA runtime load this
// library's device code onto the GPU (and so allocate): it belongs outside any region where
// allocation is forbidden, and before any stream capture.
fb_status static_scratch_for_current_device(float **out, int *sm_count) {
  int dev = -1;
  FB_CUDA_OK(cudaGetDevice(&dev));
  FB_REQUIRE(dev >= 0 && dev < kMaxDevices, FB_RUNTIME_FAILURE, "device ordinal out of range");
  std::lock_guard<std::mutex> lock(g_static_scratch_mutex);
  if (!g_static_scratch_ptr[dev]) {
    void *p = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&p, g_wgrad_static_scratch);
    if (e != cudaSuccess || p == nullptr)
      return fail(FB_RUNTIME_FAILURE,
                  std::string("cudaGetSymbolAddress(static wgrad scratch): ") + cudaGetErrorString(e));
    int sms = 0;
    e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (e != cudaSuccess || sms <= 0)
      return fail(FB_RUNTIME_FAILURE, std::string("cudaDeviceGetAttribute(SM count): ") + cudaGetErrorString(e));
    g_static_sm_count[dev] = sms;
    g_static_scratch_ptr[dev] = static_cast<float *>(p);
  }
  *out = g_static_scratch_ptr[dev];
  *sm_count = g_static_sm_count[dev];
  return FB_OK;
}

} // namespace
} // namespace fb

FB_EXPORT size_t fb_conv_wgrad_static_scratch_bytes(void) { return fb::kStaticScratchBytes; }

FB_EXPORT fb_status fb_conv_wgrad_static(void *stream, const void *dy, const void *x, void *dw, int32_t dtype,
                                         int32_t n, int32_t c, int32_t h, int32_t w, int32_t k, int32_t r,
                                         int32_t s, int32_t pad_h, int32_t pad_w, int32_t stride_h,
                                         int32_t stride_w, int32_t dil_h, int32_t dil_w, int32_t groups) {
  using namespace fb;
  clear_error();
  FB_REQUIRE(dy && x && dw, FB_INVALID_ARGUMENT, "fb_conv_wgrad_static: NULL tensor pointer");
  FB_REQUIRE(dtype == FB_DT_HALF || dtype == FB_DT_BFLOAT16 || dtype == FB_DT_FLOAT, FB_NOT_IMPLEMENTED,
             "fb_conv_wgrad_static: dtype must be f16, bf16 or f32");
  FB_REQUIRE(n > 0 && c > 0 && h > 0 && w > 0 && k > 0 && r > 0 && s > 0 && groups > 0 && stride_h > 0 &&
                 stride_w > 0 && dil_h > 0 && dil_w > 0 && pad_h >= 0 && pad_w >= 0,
             FB_INVALID_ARGUMENT, "fb_conv_wgrad_static: non-positive extent");
  FB_REQUIRE(c % groups == 0 && k % groups == 0, FB_INVALID_ARGUMENT,
             "fb_conv_wgrad_static: channels must be divisible by groups");
  const int64_t oh = 1 + ((int64_t)h + 2 * pad_h - (int64_t)(r - 1) * dil_h - 1) / stride_h;
  const int64_t ow = 1 + ((int64_t)w + 2 * pad_w - (int64_t)(s - 1) * dil_w - 1) / stride_w;
  FB_REQUIRE(oh > 0 && ow > 0, FB_INVALID_ARGUMENT, "fb_conv_wgrad_static: empty output extent");
  const int64_t cg = c / groups, kg = k / groups;
  const int64_t dw_elems = (int64_t)k * cg * r * s;
  const int64_t red = (int64_t)n * oh * ow;
  FB_REQUIRE(red < (1ll << 31) && dw_elems < (1ll << 31), FB_NOT_IMPLEMENTED,
             "fb_conv_wgrad_static: problem extent exceeds 2^31");
  float *scratch = nullptr;
  int sms = 0;
  fb_status st = static_scratch_for_current_device(&scratch, &sms);
  if (st != FB_OK) return st;
  // Same split heuristic as the planned path, then capped by the fixed scratch.
  const int64_t tiles = ((kg + BM - 1) / BM) * ((cg * r * s + BN - 1) / BN) * groups;
  int64_t split = (2 * sms + tiles - 1) / tiles;
  split = std::min<int64_t>(split, std::max<int64_t>(red / 256, 1));
  split = std::min<int64_t>(split, 64);
  const int64_t max_split = (int64_t)(kStaticScratchBytes / sizeof(float)) / dw_elems;
  FB_REQUIRE(max_split >= 1, FB_INVALID_ARGUMENT,
             "fb_conv_wgrad_static: weight gradient of " + std::to_string(dw_elems * 4) +
                 " bytes (fp32) exceeds the static scratch of " + std::to_string(kStaticScratchBytes) +
                 " bytes; use the planned path with a caller-provided workspace");
  split = std::max<int64_t>(1, std::min(split, max_split));

  static thread_local ContractParams p;
  memset(&p, 0, sizeof(p));
  p.mode = CM_WGRAD;
  p.a = dy; p.b = x; p.out = dw;
  p.a_dtype = p.b_dtype = dtype;
  p.epi.num_ops = 0;
  p.epi.acc_round_dtype = dtype;
  p.epi.out_dtype = dtype;
  p.epi.out_rank = 4;
  ConvGeomDev &g = p.g;
  g.nsp = 2;
  g.N = n; g.C = c; g.D = 1; g.H = h; g.W = w;
  g.K = k; g.Cg = (int32_t)cg; g.Kg = (int32_t)kg; g.T = 1; g.R = r; g.S = s;
  g.OD = 1; g.OH = (int32_t)oh; g.OW = (int32_t)ow;
  g.pd = 0; g.ph = pad_h; g.pw = pad_w;
  g.sd = 1; g.sh = stride_h; g.sw = stride_w;
  g.dd = 1; g.dh = dil_h; g.dw = dil_w;
  g.chan_fastest = 1;
  // dense channels-last tensors: element strides for (n, c, d, h, w)
  g.xs[0] = (int64_t)h * w * c; g.xs[1] = 1; g.xs[2] = 0; g.xs[3] = (int64_t)w * c; g.xs[4] = c;
  g.ys[0] = oh * ow * k; g.ys[1] = 1; g.ys[2] = 0; g.ys[3] = ow * k; g.ys[4] = k;
  g.ws[0] = (int64_t)r * s * cg; g.ws[1] = 1; g.ws[2] = 0; g.ws[3] = (int64_t)s * cg; g.ws[4] = cg;
  p.G = groups;
  p.M = kg; p.N = cg * r * s; p.K = red;
  p.a_kfast = 0; p.b_nfast = 1;
  p.split_k = (int32_t)split;
  p.k_chunk = ((p.K + p.split_k - 1) / p.split_k + BK - 1) / BK * BK;
  // Every element of partial[split][G][M][N] is written by the first kernel before the
  // second reads it, so the array's previous contents never matter.
  p.partial = split > 1 ? scratch : nullptr;
  dim3 grid((unsigned)((p.M + BM - 1) / BM), (unsigned)((p.N + BN - 1) / BN), (unsigned)(p.G * p.split_k));
  FB_REQUIRE(grid.y <= 65535 && grid.z <= 65535, FB_NOT_IMPLEMENTED,
             "fb_conv_wgrad_static: problem too large for one launch");
  cudaStream_t cs = static_cast<cudaStream_t>(stream);
  contract_simt_kernel<<<grid, 256, 0, cs>>>(p);
  if (p.split_k > 1) {
    int64_t total = (int64_t)p.G * p.M * p.N;
    int blocks = (int)std::min<int64_t>((total + 255) / 256, (int64_t)sms * 8);
    contract_splitk_reduce_kernel<<<blocks, 256, 0, cs>>>(p);
  }
  cudaError_t le = cudaGetLastError();
  if (le != cudaSuccess)
    return fail(FB_RUNTIME_FAILURE, std::string("fb_conv_wgrad_static: launch failed: ") + cudaGetErrorString(le));
  return FB_OK;
}
