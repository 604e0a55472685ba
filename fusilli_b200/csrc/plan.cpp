// Graph -> kernel plan lowering, artifact (de)serialisation and plan statistics.
//
// Stands where the reference runs the IREE compiler on emitted MLIR
// (include/fusilli/graph/graph.h:492-549): a validated graph becomes a list of
// kernel launches. A conv/matmul followed by a chain of pointwise nodes whose
// intermediates are virtual becomes ONE kernel with a fused epilogue (the
// reference's compile statistics expect the same fusion: "dispatch-count": 1 for
// conv+bias+relu, tests/lit/test_conv_asm_emitter_nhwc_krsc_with_relu.cpp:103-106).
// Every other node is one kernel; virtual tensors that cross kernels live in the
// caller-provided workspace.
#include <algorithm>
#include <cstring>
#include <sstream>
#include <utility>
#include <vector>

#include "common.h"

namespace fb {

static bool is_float_dt(int dt) { return dt == FB_DT_HALF || dt == FB_DT_BFLOAT16 || dt == FB_DT_FLOAT; }

static int pw_arity(int mode) {
  switch (mode) {
  case FB_PW_BINARY_SELECT: return 3;
  case FB_PW_ADD: case FB_PW_ADD_SQUARE: case FB_PW_CMP_EQ: case FB_PW_CMP_GE: case FB_PW_CMP_GT:
  case FB_PW_CMP_LE: case FB_PW_CMP_LT: case FB_PW_CMP_NEQ: case FB_PW_DIV:
  case FB_PW_GELU_APPROX_TANH_BWD: case FB_PW_GELU_BWD: case FB_PW_LOGICAL_AND:
  case FB_PW_LOGICAL_OR: case FB_PW_MAX_OP: case FB_PW_MIN_OP: case FB_PW_MUL: case FB_PW_RELU_BWD:
  case FB_PW_SUB: case FB_PW_SWISH_BWD: case FB_PW_TANH_BWD: return 2;
  default: return 1;
  }
}

static bool same_dims(const TensorInfo &a, const TensorInfo &b) {
  if (a.rank != b.rank) return false;
  for (int i = 0; i < a.rank; ++i)
    if (a.dims[i] != b.dims[i]) return false;
  return true;
}

// Dims 1.. form one dense block (in any order) and dim 0 strides over whole blocks.
static bool dense_batch_outermost(const TensorInfo &t) {
  std::vector<std::pair<int64_t, int64_t>> inner; // (stride, dim)
  for (int i = 1; i < t.rank; ++i)
    if (t.dims[i] > 1) inner.emplace_back(t.strides[i], t.dims[i]);
  std::sort(inner.begin(), inner.end());
  int64_t expect = 1;
  for (const auto &sd : inner) {
    if (sd.first != expect) return false;
    expect *= sd.second;
  }
  return t.dims[0] == 1 || t.strides[0] == expect;
}

// `o` broadcasts (right aligned) to `full` without enlarging it.
static bool broadcasts_to(const TensorInfo &o, const TensorInfo &full) {
  if (o.rank > full.rank) return false;
  for (int i = 0; i < o.rank; ++i) {
    int64_t od = o.dims[o.rank - 1 - i], fd = full.dims[full.rank - 1 - i];
    if (od != 1 && od != fd) return false;
  }
  return true;
}

static fb_status check_node(const Plan &p, int ni) {
  const fb_node_desc &d = p.nodes[ni].d;
  const std::string &nm = p.nodes[ni].name;
  auto dt = [&](int id) { return id >= 0 ? p.tensors[id].dtype : FB_DT_NOT_SET; };
  switch (d.op) {
  case FB_OP_CONV_FPROP:
  case FB_OP_CONV_DGRAD:
  case FB_OP_CONV_WGRAD: {
    FB_REQUIRE(d.num_spatial >= 1 && d.num_spatial <= 3, FB_NOT_IMPLEMENTED,
               "node '" + nm + "': convolutions with " + std::to_string(d.num_spatial) +
                   " spatial dims are not supported");
    for (int id : {d.inputs[0], d.inputs[1], d.outputs[0]}) {
      FB_REQUIRE(id >= 0, FB_INVALID_ARGUMENT, "node '" + nm + "': missing conv tensor");
      FB_REQUIRE(is_float_dt(dt(id)), FB_NOT_IMPLEMENTED,
                 "node '" + nm + "': conv tensors must be f16, bf16 or f32");
      FB_REQUIRE(p.tensors[id].rank == d.num_spatial + 2, FB_INVALID_ARGUMENT,
                 "node '" + nm + "': conv tensor rank does not match spatial dims");
    }
    for (int k = 0; k < d.num_spatial; ++k)
      FB_REQUIRE(d.stride[k] >= 1 && d.dilation[k] >= 1 && d.padding[k] >= 0, FB_INVALID_ARGUMENT,
                 "node '" + nm + "': conv stride/dilation must be >= 1 and padding >= 0");
    return FB_OK;
  }
  case FB_OP_MATMUL:
    for (int id : {d.inputs[0], d.inputs[1], d.outputs[0]}) {
      FB_REQUIRE(id >= 0, FB_INVALID_ARGUMENT, "node '" + nm + "': missing matmul tensor");
      FB_REQUIRE(is_float_dt(dt(id)) || (dt(id) == FB_DT_INT4 && id != d.outputs[0]), FB_NOT_IMPLEMENTED,
                 "node '" + nm + "': matmul on " + dtype_name(dt(id)) +
                     " tensors is not supported (f16, bf16, f32; si4 operands)");
    }
    {
      // The reference lets a batch dim of one operand divide the other's (matmul_node.h:140-150):
      // the smaller operand is read modulo its own extent.
      const TensorInfo &a = p.tensors[d.inputs[0]], &b = p.tensors[d.inputs[1]], &c = p.tensors[d.outputs[0]];
      FB_REQUIRE(a.rank >= 2 && a.rank == b.rank && a.rank == c.rank, FB_INVALID_ARGUMENT,
                 "node '" + nm + "': matmul tensors must have one rank >= 2");
      FB_REQUIRE(a.rank - 2 <= 6, FB_NOT_IMPLEMENTED, "node '" + nm + "': more than 6 matmul batch dims");
      for (int i = 0; i + 2 < a.rank; ++i)
        FB_REQUIRE(c.dims[i] % a.dims[i] == 0 && c.dims[i] % b.dims[i] == 0, FB_INVALID_ARGUMENT,
                   "node '" + nm + "': matmul batch dim " + std::to_string(i) +
                       " of an operand does not divide the result's");
    }
    return FB_OK;
  case FB_OP_SDPA:
    for (int id : {d.inputs[0], d.inputs[1], d.inputs[2], d.outputs[0]}) {
      FB_REQUIRE(id >= 0, FB_INVALID_ARGUMENT, "node '" + nm + "': missing SDPA tensor");
      FB_REQUIRE(is_float_dt(dt(id)), FB_NOT_IMPLEMENTED,
                 "node '" + nm + "': SDPA tensors must be f16, bf16 or f32");
      FB_REQUIRE(p.tensors[id].rank == 4, FB_INVALID_ARGUMENT, "node '" + nm + "': SDPA tensors must be rank 4");
    }
    if (d.inputs[3] >= 0)
      FB_REQUIRE(is_float_dt(dt(d.inputs[3])), FB_NOT_IMPLEMENTED,
                 "node '" + nm + "': SDPA mask must be f16, bf16 or f32 (additive)");
    FB_REQUIRE(d.fparams[1] == 0.f, FB_NOT_IMPLEMENTED,
               "node '" + nm + "': SDPA dropout > 0 is not supported");
    return FB_OK;
  case FB_OP_LAYERNORM:
  case FB_OP_RMSNORM: {
    FB_REQUIRE(d.inputs[0] >= 0 && d.outputs[0] >= 0, FB_INVALID_ARGUMENT, "node '" + nm + "': missing X or Y");
    int eps = d.op == FB_OP_LAYERNORM ? d.inputs[3] : d.inputs[2];
    FB_REQUIRE(eps >= 0 && p.tensors[eps].role == FB_TENSOR_SCALAR, FB_INVALID_ARGUMENT,
               "node '" + nm + "': epsilon must be a scalar constant");
    FB_REQUIRE(is_float_dt(dt(d.inputs[0])) && is_float_dt(dt(d.outputs[0])), FB_NOT_IMPLEMENTED,
               "node '" + nm + "': normalisation tensors must be f16, bf16 or f32");
    FB_REQUIRE(!(d.op == FB_OP_RMSNORM && (d.flags & FB_FLAG_NORM_TRAINING)), FB_NOT_IMPLEMENTED,
               "RmsNorm training forward phase is not implemented");
    // The kernels walk a sample as one dense run of prod(dims[1:]) elements: X and Y must be dense
    // with the batch dim outermost in memory (contiguous and channels-last both are).
    for (int id : {d.inputs[0], d.outputs[0]})
      FB_REQUIRE(dense_batch_outermost(p.tensors[id]), FB_NOT_IMPLEMENTED,
                 "node '" + nm + "': tensor '" + p.tensors[id].name +
                     "' must be dense with the batch dim outermost in memory");
    return FB_OK;
  }
  case FB_OP_BATCHNORM: {
    FB_REQUIRE(d.inputs[0] >= 0 && d.outputs[0] >= 0, FB_INVALID_ARGUMENT, "node '" + nm + "': missing X or Y");
    FB_REQUIRE(d.inputs[5] >= 0 && p.tensors[d.inputs[5]].role == FB_TENSOR_SCALAR, FB_INVALID_ARGUMENT,
               "node '" + nm + "': epsilon must be a scalar constant");
    const TensorInfo &x = p.tensors[d.inputs[0]];
    FB_REQUIRE(x.rank >= 2 && same_dims(x, p.tensors[d.outputs[0]]), FB_INVALID_ARGUMENT,
               "node '" + nm + "': X and Y must have one shape of rank >= 2");
    for (int id : {d.inputs[0], d.inputs[1], d.inputs[2], d.inputs[3], d.inputs[4], d.outputs[0], d.outputs[1],
                   d.outputs[2]}) {
      if (id < 0) continue;
      FB_REQUIRE(is_float_dt(dt(id)), FB_NOT_IMPLEMENTED,
                 "node '" + nm + "': batch normalisation tensors must be f16, bf16 or f32");
      if (id != d.inputs[0] && id != d.outputs[0])
        FB_REQUIRE(p.tensors[id].rank == 1 && p.tensors[id].dims[0] == x.dims[1] && p.tensors[id].strides[0] == 1,
                   FB_INVALID_ARGUMENT, "node '" + nm + "': per-channel tensors must be dense [C]");
    }
    if (!(d.flags & FB_FLAG_NORM_TRAINING))
      FB_REQUIRE(d.inputs[3] >= 0 && d.inputs[4] >= 0, FB_INVALID_ARGUMENT,
                 "node '" + nm + "': inference needs the running MEAN and VAR");
    return FB_OK;
  }
  case FB_OP_REDUCTION:
    FB_REQUIRE(d.mode > FB_RED_NOT_SET && d.mode < FB_RED_MODE_COUNT, FB_INVALID_ARGUMENT,
               "node '" + nm + "': bad reduction mode");
    FB_REQUIRE(d.inputs[0] >= 0 && d.outputs[0] >= 0, FB_INVALID_ARGUMENT, "node '" + nm + "': missing X or Y");
    return FB_OK;
  case FB_OP_POINTWISE: {
    FB_REQUIRE(d.mode > FB_PW_NOT_SET && d.mode < FB_PW_MODE_COUNT, FB_INVALID_ARGUMENT,
               "node '" + nm + "': bad pointwise mode");
    int ar = pw_arity(d.mode);
    for (int k = 0; k < ar; ++k)
      FB_REQUIRE(d.inputs[k] >= 0, FB_INVALID_ARGUMENT, "node '" + nm + "': missing pointwise input");
    FB_REQUIRE(d.outputs[0] >= 0, FB_INVALID_ARGUMENT, "node '" + nm + "': missing pointwise output");
    for (int k = 0; k < ar; ++k)
      FB_REQUIRE(broadcasts_to(p.tensors[d.inputs[k]], p.tensors[d.outputs[0]]), FB_INVALID_ARGUMENT,
                 "node '" + nm + "': input does not broadcast to the output shape");
    return FB_OK;
  }
  default:
    return fail(FB_NOT_IMPLEMENTED, "node '" + nm + "': operation is not supported by the B200 backend");
  }
}

fb_status lower(Plan &p) {
  const int nt = (int)p.tensors.size(), nn = (int)p.nodes.size();
  // Int4 exists only as a bound matmul operand (weight-only quantisation, the reference's
  // samples/matmul/matmul_int4_fp16.cpp); every other use needs byte-addressable elements.
  std::vector<bool> matmul_operand_only(nt, true), used(nt, false);
  for (const NodeInfo &n : p.nodes) {
    for (int k = 0; k < FB_MAX_NODE_INPUTS; ++k) {
      const int id = n.d.inputs[k];
      if (id < 0 || id >= nt) continue;
      used[id] = true;
      if (n.d.op != FB_OP_MATMUL || k > 1) matmul_operand_only[id] = false;
    }
    for (int k = 0; k < FB_MAX_NODE_OUTPUTS; ++k)
      if (n.d.outputs[k] >= 0 && n.d.outputs[k] < nt) matmul_operand_only[n.d.outputs[k]] = false;
  }
  for (int i = 0; i < nt; ++i) {
    const TensorInfo &t = p.tensors[i];
    const bool ok = dtype_size(t.dtype) > 0 ||
                    (t.dtype == FB_DT_INT4 && t.role == FB_TENSOR_INPUT && used[i] && matmul_operand_only[i]);
    FB_REQUIRE(ok, FB_NOT_IMPLEMENTED,
               "tensor '" + t.name + "': data type " + dtype_name(t.dtype) +
                   (t.dtype == FB_DT_INT4 ? " is supported only as an input operand of a matmul"
                                          : " is not supported by the B200 backend"));
  }
  std::vector<int> uses(nt, 0);
  std::vector<std::vector<int>> consumers(nt);
  for (int i = 0; i < nn; ++i) {
    fb_status st = check_node(p, i);
    if (st != FB_OK) return st;
    for (int k = 0; k < FB_MAX_NODE_INPUTS; ++k) {
      int id = p.nodes[i].d.inputs[k];
      if (id >= 0) {
        uses[id]++;
        consumers[id].push_back(i);
      }
    }
  }
  std::vector<bool> consumed(nn, false);
  p.steps.clear();
  for (int i = 0; i < nn; ++i) {
    if (consumed[i]) continue;
    consumed[i] = true;
    const fb_node_desc &d = p.nodes[i].d;
    Step s;
    s.node = i;
    s.out_tensor = d.outputs[0];
    switch (d.op) {
    case FB_OP_CONV_FPROP:
    case FB_OP_CONV_DGRAD:
    case FB_OP_CONV_WGRAD:
    case FB_OP_MATMUL: {
      s.kind = STEP_CONTRACT;
      int cur = d.outputs[0];
      while (s.num_epilogue < kMaxEpilogueOps) {
        const TensorInfo &ct = p.tensors[cur];
        if (ct.role != FB_TENSOR_VIRTUAL || uses[cur] != 1) break;
        int pi = consumers[cur][0];
        const fb_node_desc &pd = p.nodes[pi].d;
        if (pd.op != FB_OP_POINTWISE || consumed[pi] || pi < i) break;
        int ar = pw_arity(pd.mode);
        if (ar == 3) break;
        const TensorInfo &ot = p.tensors[pd.outputs[0]];
        if (!same_dims(ot, ct) || !is_float_dt(ot.dtype)) break;
        EpilogueOpInfo op;
        op.mode = pd.mode;
        op.out_tensor = pd.outputs[0];
        memcpy(op.fparams, pd.fparams, sizeof(op.fparams));
        if (ar == 2) {
          bool v_in0 = pd.inputs[0] == cur;
          int other = v_in0 ? pd.inputs[1] : pd.inputs[0];
          if (other == cur) break; // x op x
          const TensorInfo &o = p.tensors[other];
          if (o.role != FB_TENSOR_INPUT && o.role != FB_TENSOR_SCALAR) break;
          if (!broadcasts_to(o, ct)) break;
          op.operand = other;
          op.value_is_in1 = v_in0 ? 0 : 1;
        }
        s.epilogue[s.num_epilogue++] = op;
        consumed[pi] = true;
        cur = pd.outputs[0];
      }
      s.out_tensor = cur;
      if (d.op == FB_OP_CONV_WGRAD) {
        // Reduction over N*spatial is long and the output small: split it over
        // CTAs, fp32 partials in the workspace, reduced in a fixed order.
        const TensorInfo &dy = p.tensors[d.inputs[0]];
        const TensorInfo &dw = p.tensors[d.outputs[0]];
        int64_t red = dy.dims[0];
        for (int k = 2; k < dy.rank; ++k) red *= dy.dims[k];
        int64_t dw_elems = 1;
        for (int k = 0; k < dw.rank; ++k) dw_elems *= dw.dims[k];
        int64_t kout = dw.dims[0], ncols = dw_elems / kout;
        int64_t tiles = ((kout + 63) / 64) * ((ncols + 63) / 64);
        int64_t split = (2 * 148 + tiles - 1) / tiles;
        int64_t max_split = red / 256;
        if (split > max_split) split = max_split;
        if (split > 64) split = 64;
        if (split < 1) split = 1;
        s.split_k = (int32_t)split;
        if (s.split_k > 1) s.scratch_bytes = (int64_t)s.split_k * dw_elems * 4;
      }
      if (d.op == FB_OP_MATMUL)
        s.engine = gemm_tc_eligible(p, s) ? ENGINE_TCGEN05 : ENGINE_SIMT;
      else if (d.op == FB_OP_CONV_WGRAD)
        s.engine = conv_wgrad_tc_eligible(p, s) ? ENGINE_TCGEN05 : ENGINE_SIMT;
      else
        s.engine = conv_tc_eligible(p, s) ? ENGINE_TCGEN05
                                          : (conv_split_f32_eligible(p, s) ? ENGINE_TCGEN05_SPLIT : ENGINE_SIMT);
      if (s.engine == ENGINE_TCGEN05_SPLIT) {
        s.split_k = 1;
        s.scratch_bytes = conv_split_f32_scratch_bytes(p, s);
      }
      if (s.engine == ENGINE_TCGEN05) {
        // (a smaller shape of a dynamic plan may fall to the CUDA-core kernel: keep its partials' room too)
        const int64_t simt_bytes = d.op == FB_OP_CONV_WGRAD ? s.scratch_bytes : 0;
        s.split_k = 1;
        s.scratch_bytes = 0;
        if (d.op == FB_OP_CONV_WGRAD)
          s.scratch_bytes = std::max(conv_wgrad_tc_scratch_bytes(p, s, &s.split_k), simt_bytes);
      }
      break;
    }
    case FB_OP_SDPA:
      s.kind = STEP_SDPA;
      s.engine = sdpa_tc_eligible(p, s) ? ENGINE_TCGEN05 : ENGINE_SIMT;
      break;
    case FB_OP_LAYERNORM:
    case FB_OP_RMSNORM: s.kind = STEP_NORM; break;
    case FB_OP_BATCHNORM:
      s.kind = STEP_BATCHNORM;
      s.scratch_bytes = batchnorm_scratch_bytes(p, s, &s.split_k);
      break;
    case FB_OP_REDUCTION: s.kind = STEP_REDUCTION; break;
    case FB_OP_POINTWISE: s.kind = STEP_POINTWISE; break;
    default: return fail(FB_INTERNAL_ERROR, "lower: unexpected op");
    }
    p.steps.push_back(s);
  }
  // Workspace: virtual tensors written by one kernel and read by another, then
  // per-step scratch. 256-byte aligned bump allocation, no reuse.
  size_t off = 0;
  auto place = [&](int id) {
    if (id < 0) return;
    TensorInfo &t = p.tensors[id];
    if (t.role != FB_TENSOR_VIRTUAL || t.ws_offset >= 0) return;
    t.ws_offset = (int64_t)off;
    off += ((size_t)t.phys_elems() * dtype_size(t.dtype) + 255) & ~(size_t)255;
  };
  for (Step &s : p.steps) {
    place(s.out_tensor);
    const fb_node_desc &d = p.nodes[s.node].d;
    if (s.kind == STEP_NORM || s.kind == STEP_BATCHNORM)
      for (int k = 1; k < FB_MAX_NODE_OUTPUTS; ++k)
        if (d.outputs[k] >= 0 && uses[d.outputs[k]] > 0) place(d.outputs[k]);
    if (s.scratch_bytes > 0) {
      s.scratch_offset = (int64_t)off;
      off += ((size_t)s.scratch_bytes + 255) & ~(size_t)255;
    }
  }
  p.workspace_bytes = off;
  return FB_OK;
}

// ---- dynamic dims --------------------------------------------------------------
// The reference marks dims as dynamic on the tensors (tensor_attributes.h:71-84): dims and strides
// stay representative, the emitted function takes `?` extents, and the buffers of each call carry
// the concrete ones. Here the plan keeps the whole graph, so a call with new extents re-derives
// the shapes and lowers again.

// Dense strides for `t.dims` in the layout order of the representative strides (innermost =
// smallest stride; among equal strides, which only unit dims have, the later dim is inner).
static void restride(TensorInfo &t) {
  int order[FB_MAX_RANK];
  for (int i = 0; i < t.rank; ++i) order[i] = i;
  for (int i = 1; i < t.rank; ++i)
    for (int j = i; j > 0; --j) {
      const int a = order[j - 1], b = order[j];
      const bool b_inner = t.strides[b] < t.strides[a] || (t.strides[b] == t.strides[a] && b > a);
      if (!b_inner) break;
      order[j - 1] = b;
      order[j] = a;
    }
  int64_t run = 1;
  for (int i = 0; i < t.rank; ++i) {
    t.strides[order[i]] = run;
    run *= t.dims[order[i]];
  }
}

// Extent of dim `k` of output `slot` of node `d` as its inputs imply it, -1 when the node gives
// no rule (the reference makes the user state dX and dW dims, conv_node.h:546-559).
static int64_t implied_out_dim(const Plan &p, const fb_node_desc &d, int slot, int k) {
  auto T = [&](int id) -> const TensorInfo & { return p.tensors[id]; };
  switch (d.op) {
  case FB_OP_CONV_FPROP: {
    const TensorInfo &x = T(d.inputs[0]), &w = T(d.inputs[1]);
    if (k == 0) return x.dims[0];
    if (k == 1) return w.dims[0];
    const int s = k - 2;
    return 1 + (x.dims[k] + 2 * d.padding[s] - (w.dims[k] - 1) * d.dilation[s] - 1) / d.stride[s];
  }
  case FB_OP_CONV_DGRAD: return k == 0 ? T(d.inputs[0]).dims[0] : -1;
  case FB_OP_CONV_WGRAD: return -1;
  case FB_OP_MATMUL: {
    const TensorInfo &a = T(d.inputs[0]), &b = T(d.inputs[1]);
    const int r = T(d.outputs[0]).rank;
    if (a.rank != r || b.rank != r) return -1;
    if (k == r - 2) return a.dims[r - 2];
    if (k == r - 1) return b.dims[r - 1];
    return a.dims[k] > b.dims[k] ? a.dims[k] : b.dims[k];
  }
  case FB_OP_SDPA: return k == 3 ? T(d.inputs[2]).dims[3] : T(d.inputs[0]).dims[k];
  case FB_OP_LAYERNORM:
  case FB_OP_RMSNORM:
    if (slot == 0 || k == 0) return T(d.inputs[0]).dims[k];
    return 1;
  case FB_OP_BATCHNORM: return slot == 0 ? T(d.inputs[0]).dims[k] : T(d.inputs[0]).dims[1];
  case FB_OP_REDUCTION: return T(d.inputs[0]).dims[k]; // a dynamic dim is never a reduced one
  case FB_OP_POINTWISE: {
    const int r = T(d.outputs[0]).rank;
    int64_t v = 1;
    for (int i = 0; i < FB_MAX_NODE_INPUTS; ++i) {
      if (d.inputs[i] < 0) continue;
      const TensorInfo &in = T(d.inputs[i]);
      const int idx = k - (r - in.rank);
      if (idx >= 0 && in.dims[idx] > v) v = in.dims[idx];
    }
    return v;
  }
  default: return -1;
  }
}

// What validate() checked on the representative shape and a new extent can break.
static fb_status check_runtime_shapes(const Plan &p, const NodeInfo &n) {
  const fb_node_desc &d = n.d;
  auto T = [&](int id) -> const TensorInfo & { return p.tensors[id]; };
  auto bad = [&](const std::string &what) {
    return fail(FB_INVALID_ARGUMENT, "node '" + n.name + "': runtime shapes disagree: " + what);
  };
  switch (d.op) {
  case FB_OP_CONV_FPROP:
  case FB_OP_CONV_DGRAD:
  case FB_OP_CONV_WGRAD: {
    // (image, filter, result) in fprop roles: fprop X,W,Y; dgrad DX,W,DY; wgrad X,DW,DY
    const TensorInfo &img = d.op == FB_OP_CONV_FPROP ? T(d.inputs[0]) : (d.op == FB_OP_CONV_DGRAD ? T(d.outputs[0]) : T(d.inputs[1]));
    const TensorInfo &flt = d.op == FB_OP_CONV_WGRAD ? T(d.outputs[0]) : T(d.inputs[1]);
    const TensorInfo &res = d.op == FB_OP_CONV_FPROP ? T(d.outputs[0]) : T(d.inputs[0]);
    if (img.dims[0] != res.dims[0]) return bad("batch sizes differ");
    for (int k = 2; k < img.rank; ++k) {
      const int s = k - 2;
      const int64_t want = 1 + (img.dims[k] + 2 * d.padding[s] - (flt.dims[k] - 1) * d.dilation[s] - 1) / d.stride[s];
      if (want != res.dims[k]) return bad("spatial dim " + std::to_string(s) + " of the convolution result");
    }
    return FB_OK;
  }
  case FB_OP_MATMUL: {
    const TensorInfo &a = T(d.inputs[0]), &b = T(d.inputs[1]);
    if (a.dims[a.rank - 1] != b.dims[b.rank - 2]) return bad("matmul K");
    for (int k = 0; k + 2 < a.rank && a.rank == b.rank; ++k)
      if (a.dims[k] != b.dims[k] && a.dims[k] != 1 && b.dims[k] != 1 && a.dims[k] % b.dims[k] != 0 &&
          b.dims[k] % a.dims[k] != 0)
        return bad("matmul batch dims");
    return FB_OK;
  }
  case FB_OP_SDPA: {
    const TensorInfo &q = T(d.inputs[0]), &k = T(d.inputs[1]), &v = T(d.inputs[2]);
    if (q.dims[0] != k.dims[0] || q.dims[0] != v.dims[0]) return bad("SDPA batch");
    if (k.dims[2] != v.dims[2]) return bad("SDPA key and value sequence lengths");
    if (q.dims[3] != k.dims[3]) return bad("SDPA head dim");
    if (d.inputs[3] >= 0) {
      const TensorInfo &m = T(d.inputs[3]);
      const int64_t full[4] = {q.dims[0], q.dims[1], q.dims[2], k.dims[2]};
      for (int i = 0; i < 4; ++i)
        if (m.dims[i] != 1 && m.dims[i] != full[i]) return bad("SDPA mask");
    }
    return FB_OK;
  }
  case FB_OP_LAYERNORM:
  case FB_OP_RMSNORM: {
    const TensorInfo &x = T(d.inputs[0]);
    const int nparams = d.op == FB_OP_LAYERNORM ? 2 : 1;
    for (int i = 1; i <= nparams; ++i) {
      if (d.inputs[i] < 0) continue;
      const TensorInfo &g = T(d.inputs[i]);
      for (int k = 1; k < x.rank && g.rank == x.rank; ++k)
        if (g.dims[k] != x.dims[k]) return bad("normalisation scale / bias");
    }
    return FB_OK;
  }
  default: return FB_OK; // pointwise broadcasting is re-checked by the lowering
  }
}

fb_status specialize(const Plan &base, const int64_t *arg_dims, Plan &out) {
  FB_REQUIRE(arg_dims != nullptr, FB_INVALID_ARGUMENT, "runtime dims are NULL");
  out = base;
  out.steps.clear();
  for (TensorInfo &t : out.tensors) t.ws_offset = -1;
  for (int a = 0; a < out.num_args; ++a) {
    TensorInfo &t = out.tensors[out.arg_tensor[a]];
    const int64_t *rt = arg_dims + (size_t)a * FB_MAX_RANK;
    for (int k = 0; k < t.rank; ++k) {
      FB_REQUIRE(rt[k] >= 1, FB_INVALID_ARGUMENT,
                 "tensor '" + t.name + "': runtime dim " + std::to_string(k) + " is " + std::to_string(rt[k]));
      if (t.dynamic_mask >> k & 1) continue;
      FB_REQUIRE(rt[k] == t.dims[k], FB_INVALID_ARGUMENT,
                 "tensor '" + t.name + "': dim " + std::to_string(k) + " is static (" + std::to_string(t.dims[k]) +
                     ") but the buffer has " + std::to_string(rt[k]));
    }
    if (t.dynamic_mask) {
      for (int k = 0; k < t.rank; ++k) t.dims[k] = rt[k];
      restride(t);
    }
  }
  for (const NodeInfo &n : out.nodes) {
    for (int slot = 0; slot < FB_MAX_NODE_OUTPUTS; ++slot) {
      const int id = n.d.outputs[slot];
      if (id < 0 || out.tensors[id].dynamic_mask == 0) continue;
      TensorInfo &t = out.tensors[id];
      for (int k = 0; k < t.rank; ++k) {
        if (!(t.dynamic_mask >> k & 1)) continue;
        const int64_t v = implied_out_dim(out, n.d, slot, k);
        if (t.role == FB_TENSOR_VIRTUAL) {
          FB_REQUIRE(v >= 1, FB_NOT_IMPLEMENTED,
                     "node '" + n.name + "': dynamic dim " + std::to_string(k) + " of virtual tensor '" + t.name +
                         "' does not follow from the node's inputs");
          t.dims[k] = v;
        } else {
          FB_REQUIRE(v < 0 || v == t.dims[k], FB_INVALID_ARGUMENT,
                     "tensor '" + t.name + "': the buffer's dim " + std::to_string(k) + " is " +
                         std::to_string(t.dims[k]) + " but the inputs of node '" + n.name + "' imply " +
                         std::to_string(v));
        }
      }
      if (t.role == FB_TENSOR_VIRTUAL) restride(t);
    }
    fb_status st = check_runtime_shapes(out, n);
    if (st != FB_OK) return st;
  }
  return lower(out);
}

// ---- serialisation -----------------------------------------------------------
// Layout: magic[8] | abi u32 | arch u32 | payload_len u64 | fnv1a64(payload) u64 | payload

static const char kMagic[8] = {'F', 'B', '2', 'P', 'L', 'A', 'N', '\0'};
static const uint32_t kArch = 100; // sm_100a

static uint64_t fnv1a(const uint8_t *p, size_t n) {
  uint64_t h = 1469598103934665603ull;
  for (size_t i = 0; i < n; ++i) {
    h ^= p[i];
    h *= 1099511628211ull;
  }
  return h;
}

struct Writer {
  std::vector<uint8_t> b;
  template <typename T> void pod(const T &v) {
    const uint8_t *q = reinterpret_cast<const uint8_t *>(&v);
    b.insert(b.end(), q, q + sizeof(T));
  }
  void str(const std::string &s) {
    pod<uint32_t>((uint32_t)s.size());
    b.insert(b.end(), s.begin(), s.end());
  }
};

struct Reader {
  const uint8_t *p;
  size_t n, off = 0;
  bool ok = true;
  template <typename T> T pod() {
    T v{};
    if (off + sizeof(T) > n) {
      ok = false;
      return v;
    }
    memcpy(&v, p + off, sizeof(T));
    off += sizeof(T);
    return v;
  }
  std::string str() {
    uint32_t len = pod<uint32_t>();
    if (!ok || off + len > n) {
      ok = false;
      return "";
    }
    std::string s(reinterpret_cast<const char *>(p + off), len);
    off += len;
    return s;
  }
};

fb_status serialize(const Plan &p, std::vector<uint8_t> &out) {
  Writer w;
  w.str(p.name);
  w.pod<uint32_t>((uint32_t)p.tensors.size());
  for (const TensorInfo &t : p.tensors) {
    w.str(t.name);
    w.pod(t.dtype); w.pod(t.role); w.pod(t.rank); w.pod(t.arg_index);
    for (int i = 0; i < FB_MAX_RANK; ++i) w.pod(t.dims[i]);
    for (int i = 0; i < FB_MAX_RANK; ++i) w.pod(t.strides[i]);
    w.pod(t.scalar);
    w.pod(t.dynamic_mask);
    w.pod(t.ws_offset);
  }
  w.pod<uint32_t>((uint32_t)p.nodes.size());
  for (const NodeInfo &nd : p.nodes) {
    w.str(nd.name);
    fb_node_desc d = nd.d;
    d.name = nullptr;
    w.pod(d);
  }
  w.pod<uint32_t>((uint32_t)p.steps.size());
  for (const Step &s : p.steps) w.pod(s);
  w.pod<int32_t>(p.num_args);
  w.pod<uint64_t>(p.workspace_bytes);
  out.clear();
  Writer h;
  for (char c : kMagic) h.pod(c);
  h.pod<uint32_t>(FB_ABI_VERSION);
  h.pod<uint32_t>(kArch);
  h.pod<uint64_t>(w.b.size());
  h.pod<uint64_t>(fnv1a(w.b.data(), w.b.size()));
  out = h.b;
  out.insert(out.end(), w.b.begin(), w.b.end());
  return FB_OK;
}

fb_status deserialize(const uint8_t *bytes, size_t n, Plan &p) {
  const size_t header = 8 + 4 + 4 + 8 + 8;
  FB_REQUIRE(n >= header && memcmp(bytes, kMagic, 8) == 0, FB_RUNTIME_FAILURE,
             "artifact is not a fusilli-b200 plan (bad magic)");
  Reader h{bytes + 8, n - 8};
  uint32_t abi = h.pod<uint32_t>(), arch = h.pod<uint32_t>();
  uint64_t len = h.pod<uint64_t>(), sum = h.pod<uint64_t>();
  FB_REQUIRE(abi == FB_ABI_VERSION, FB_RUNTIME_FAILURE,
             "artifact ABI version " + std::to_string(abi) + " does not match library version " +
                 std::to_string(FB_ABI_VERSION));
  FB_REQUIRE(arch == kArch, FB_RUNTIME_FAILURE, "artifact was built for a different architecture");
  FB_REQUIRE(len == n - header, FB_RUNTIME_FAILURE, "artifact is truncated or has trailing bytes");
  FB_REQUIRE(fnv1a(bytes + header, len) == sum, FB_RUNTIME_FAILURE, "artifact checksum mismatch");
  Reader r{bytes + header, (size_t)len};
  p.name = r.str();
  uint32_t nt = r.pod<uint32_t>();
  FB_REQUIRE(r.ok && nt < (1u << 20), FB_RUNTIME_FAILURE, "artifact payload is malformed");
  p.tensors.resize(nt);
  for (TensorInfo &t : p.tensors) {
    t.name = r.str();
    t.dtype = r.pod<int32_t>(); t.role = r.pod<int32_t>(); t.rank = r.pod<int32_t>();
    t.arg_index = r.pod<int32_t>();
    for (int i = 0; i < FB_MAX_RANK; ++i) t.dims[i] = r.pod<int64_t>();
    for (int i = 0; i < FB_MAX_RANK; ++i) t.strides[i] = r.pod<int64_t>();
    t.scalar = r.pod<double>();
    t.dynamic_mask = r.pod<uint32_t>();
    t.ws_offset = r.pod<int64_t>();
    FB_REQUIRE(r.ok && t.rank >= 1 && t.rank <= FB_MAX_RANK, FB_RUNTIME_FAILURE,
               "artifact payload is malformed");
  }
  uint32_t nn = r.pod<uint32_t>();
  FB_REQUIRE(r.ok && nn < (1u << 20), FB_RUNTIME_FAILURE, "artifact payload is malformed");
  p.nodes.resize(nn);
  for (NodeInfo &nd : p.nodes) {
    nd.name = r.str();
    nd.d = r.pod<fb_node_desc>();
    nd.d.name = nullptr;
  }
  uint32_t ns = r.pod<uint32_t>();
  FB_REQUIRE(r.ok && ns < (1u << 20), FB_RUNTIME_FAILURE, "artifact payload is malformed");
  p.steps.resize(ns);
  for (Step &s : p.steps) {
    s = r.pod<Step>();
    FB_REQUIRE(r.ok && s.node >= 0 && s.node < (int)nn && s.out_tensor >= 0 && s.out_tensor < (int)nt,
               FB_RUNTIME_FAILURE, "artifact payload is malformed");
  }
  p.num_args = r.pod<int32_t>();
  p.workspace_bytes = (size_t)r.pod<uint64_t>();
  FB_REQUIRE(r.ok && r.off == r.n, FB_RUNTIME_FAILURE, "artifact payload is malformed");
  p.arg_tensor.assign(p.num_args, -1);
  for (uint32_t i = 0; i < nt; ++i) {
    int a = p.tensors[i].arg_index;
    FB_REQUIRE(a < p.num_args, FB_RUNTIME_FAILURE, "artifact payload is malformed");
    if (a >= 0) p.arg_tensor[a] = (int)i;
  }
  for (int a = 0; a < p.num_args; ++a)
    FB_REQUIRE(p.arg_tensor[a] >= 0, FB_RUNTIME_FAILURE, "artifact payload is malformed");
  return FB_OK;
}

const char *step_kernel_name(const Plan &p, const Step &s) {
  int op = p.nodes[s.node].d.op;
  bool tc = s.engine == ENGINE_TCGEN05;
  switch (s.kind) {
  case STEP_POINTWISE: return "pointwise";
  case STEP_REDUCTION: return "reduction";
  case STEP_NORM: return op == FB_OP_LAYERNORM ? "layernorm" : "rmsnorm";
  case STEP_BATCHNORM: return "batchnorm";
  case STEP_SDPA: return tc ? "sdpa_fwd_tcgen05" : "sdpa_fwd_simt";
  case STEP_CONTRACT:
    switch (op) {
    case FB_OP_MATMUL: return tc ? "gemm_tcgen05" : "gemm_simt";
    case FB_OP_CONV_FPROP:
      if (s.engine == ENGINE_TCGEN05_SPLIT) return "conv_fprop_split_f32_tcgen05";
      return tc ? "conv_fprop_tcgen05" : "conv_fprop_simt";
    case FB_OP_CONV_DGRAD: return tc ? "conv_dgrad_tcgen05" : "conv_dgrad_simt";
    case FB_OP_CONV_WGRAD: return tc ? "conv_wgrad_tcgen05" : "conv_wgrad_simt";
    }
  }
  return "unknown";
}

int step_launches(const Plan &p, const Step &s) {
  if (s.kind == STEP_BATCHNORM) return (p.nodes[s.node].d.flags & FB_FLAG_NORM_TRAINING) ? 3 : 1;
  const bool wgrad = p.nodes[s.node].d.op == FB_OP_CONV_WGRAD;
  if (wgrad && s.engine == ENGINE_TCGEN05) return 2; // partial kernel + slice reduction
  if (s.engine == ENGINE_TCGEN05_SPLIT) return 2;    // piece split of X and W, convolution
  return s.split_k > 1 ? 2 : 1;
}

std::string stats_json(const Plan &p) {
  std::ostringstream o;
  int launches = 0;
  for (const Step &s : p.steps) launches += step_launches(p, s);
  o << "{\"name\": \"" << p.name << "\", \"dispatch-count\": " << launches
    << ", \"transient-memory-size\": " << p.workspace_bytes << ", \"steps\": [";
  for (size_t i = 0; i < p.steps.size(); ++i) {
    const Step &s = p.steps[i];
    if (i) o << ", ";
    o << "{\"kernel\": \"" << step_kernel_name(p, s) << "\", \"node\": \"" << p.nodes[s.node].name
      << "\", \"fused\": [";
    for (int k = 0; k < s.num_epilogue; ++k) {
      if (k) o << ", ";
      o << s.epilogue[k].mode;
    }
    o << "], \"split_k\": " << s.split_k << "}";
  }
  o << "]}";
  return o.str();
}

fb_status build_epilogue(const ExecContext &cx, const Step &s, EpilogueDev &e) {
  const Plan &p = *cx.plan;
  memset(&e, 0, sizeof(e));
  const fb_node_desc &d = p.nodes[s.node].d;
  const TensorInfo &acc_t = p.tensors[d.outputs[0]];
  const TensorInfo &out_t = p.tensors[s.out_tensor];
  e.num_ops = s.num_epilogue;
  e.acc_round_dtype = acc_t.dtype;
  e.out_dtype = out_t.dtype;
  e.out_rank = out_t.rank;
  for (int i = 0; i < s.num_epilogue; ++i) {
    const EpilogueOpInfo &src = s.epilogue[i];
    EpiOpDev &op = e.ops[i];
    op.mode = src.mode;
    op.value_is_in1 = src.value_is_in1;
    op.round_dtype = p.tensors[src.out_tensor].dtype;
    memcpy(op.fparams, src.fparams, sizeof(op.fparams));
    if (src.operand >= 0) {
      const TensorInfo &o = p.tensors[src.operand];
      if (o.role == FB_TENSOR_SCALAR) {
        op.operand_kind = 2;
        op.scalar = (float)o.scalar;
      } else {
        op.operand_kind = 1;
        op.operand = cx.tensor_ptr(src.operand);
        op.operand_dtype = o.dtype;
        FB_REQUIRE(op.operand != nullptr, FB_INTERNAL_ERROR, "epilogue operand has no buffer");
        for (int k = 0; k < o.rank; ++k) {
          int od = out_t.rank - o.rank + k;
          op.strides[od] = (o.dims[k] == 1) ? 0 : o.strides[k];
        }
      }
    }
  }
  return FB_OK;
}

} // namespace fb
