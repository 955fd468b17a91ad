// See plan.h. Validation mirrors what the reference checks when it matches an
// op (kernel size, strides, operand ranks) and reports INVALID_ARGUMENT /
// UNIMPLEMENTED instead of silently taking another path.
#include "plan.h"

#include <algorithm>
#include <climits>
#include <cstdarg>
#include <cstdint>
#include <cstdlib>
#include <cstring>
#include <map>
#include <memory>

#include "../../include/torq_b200.h"
#include "kernels.h"

namespace tb200 {

namespace {

struct Builder {
  const std::vector<tb200_tensor_t>& tensors;
  const std::vector<tb200_op_t>& ops;
  const std::vector<uint8_t>& constants;
  Plan& plan;
  std::string& err;
  int status = TB200_OK;

  int fail(int st, const char* fmt, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof(buf), fmt, ap);
    va_end(ap);
    err = buf;
    status = st;
    return st;
  }

  bool valid_id(int id) const { return id >= 0 && id < (int)tensors.size(); }

  size_t add_const(const void* data, size_t bytes) {
    size_t off = (plan.const_image.size() + 255) & ~(size_t)255;
    plan.const_image.resize(off + bytes);
    memcpy(plan.const_image.data() + off, data, bytes);
    return off;
  }

  // Uploads a constant tensor's bytes unchanged, once per tensor id (the tied embedding /
  // LM-head table is named by two ops).
  std::map<int, size_t> raw_offsets;
  bool add_raw_const(int id, size_t min_bytes, const char* what, int op_index, size_t& off) {
    if (!valid_id(id) || tensors[id].kind != TB200_TENSOR_CONSTANT || tensors[id].const_bytes < min_bytes) {
      fail(TB200_INVALID_ARGUMENT, "op %d: %s is not a constant of at least %zu bytes", op_index, what, min_bytes);
      return false;
    }
    auto it = raw_offsets.find(id);
    if (it == raw_offsets.end())
      it = raw_offsets.emplace(id, add_const(constants.data() + tensors[id].const_offset, tensors[id].const_bytes)).first;
    off = it->second;
    return true;
  }

  bool is_t(int id, uint32_t dtype, uint32_t rank) const {
    return valid_id(id) && tensors[id].dtype == dtype && tensors[id].rank == rank;
  }

  template <typename T>
  const T* const_data(int id, size_t min_elems, const char* what, int op_index) {
    if (!valid_id(id) || tensors[id].kind != TB200_TENSOR_CONSTANT) {
      fail(TB200_INVALID_ARGUMENT, "op %d: %s is not a constant tensor", op_index, what);
      return nullptr;
    }
    const auto& t = tensors[id];
    if (t.const_bytes < min_elems * sizeof(T)) {
      fail(TB200_INVALID_ARGUMENT, "op %d: %s holds %llu bytes, needs %zu", op_index, what,
           (unsigned long long)t.const_bytes, min_elems * sizeof(T));
      return nullptr;
    }
    return reinterpret_cast<const T*>(constants.data() + t.const_offset);
  }

  size_t numel(int id) const {
    const auto& t = tensors[id];
    size_t n = 1;
    for (uint32_t i = 0; i < t.rank; i++) n *= (size_t)t.shape[i];
    return n;
  }

  bool act_i8(int id, uint32_t rank) const {
    return valid_id(id) && tensors[id].dtype == TB200_I8 && tensors[id].rank == rank &&
           tensors[id].kind != TB200_TENSOR_CONSTANT;
  }

  // Per-channel epilogue parameters from bias[], multiplier[], shift[] of the op.
  // Mode (B) (compiler/torq/Utils/Kernel.h:607-635) becomes the same device code
  // with scale[c] = M[c] >> (S[c] - min S), shift = min S and single rounding
  // (compiler/torq/Conversions/LinalgToTorqHL/PatternUtils.cpp:3536-3549).
  bool chan_params(const tb200_op_t& op, int op_index, int OC, const int32_t* wsum, long long K,
                   bool fold_zp, std::vector<ChanParams>& out, int& double_round) {
    int nscale = op.per_channel ? OC : 1;
    const int32_t* mult = const_data<int32_t>(op.multiplier, nscale, "multiplier", op_index);
    const int8_t* shift = const_data<int8_t>(op.shift, nscale, "shift", op_index);
    if (!mult || !shift) return false;
    const int32_t* bias = nullptr;
    int bias_len = 0;
    if (op.bias >= 0) {
      if (!valid_id(op.bias)) {
        fail(TB200_INVALID_ARGUMENT, "op %d: bad bias id", op_index);
        return false;
      }
      bias_len = (int)numel(op.bias);
      if (bias_len != 1 && bias_len != OC) {
        fail(TB200_INVALID_ARGUMENT, "op %d: bias has %d entries, expected 1 or %d", op_index, bias_len, OC);
        return false;
      }
      bias = const_data<int32_t>(op.bias, bias_len, "bias", op_index);
      if (!bias) return false;
    }
    int min_shift = 127;
    for (int i = 0; i < nscale; i++) {
      if (shift[i] < 2 || shift[i] > 62) {
        fail(TB200_INVALID_ARGUMENT, "op %d: rescale shift %d outside [2,62]", op_index, (int)shift[i]);
        return false;
      }
      min_shift = std::min(min_shift, (int)shift[i]);
    }
    double_round = op.double_round;
    if (op.requant_mode == TB200_REQUANT_NPU) double_round = 0;
    else if (op.requant_mode != TB200_REQUANT_TOSA) {
      fail(TB200_INVALID_ARGUMENT, "op %d: unknown requant mode %d", op_index, op.requant_mode);
      return false;
    }
    out.resize(OC);
    last_hi_shift = true;
    last_min_shift = 64;
    last_max_shift = 0;
    for (int c = 0; c < OC; c++) {
      int i = op.per_channel ? c : 0;
      ChanParams p{};
      uint32_t b = bias ? (uint32_t)bias[bias_len == 1 ? 0 : c] : 0u;
      p.wsum = wsum ? wsum[c] : 0;
      if (fold_zp && wsum) {
        // bias - izp * sum(w) + K * izp * wzp, modulo 2^32
        b -= (uint32_t)op.in0_zp * (uint32_t)wsum[c];
        b += (uint32_t)(K & 0xffffffffll) * (uint32_t)op.in0_zp * (uint32_t)op.weight_zp;
      }
      p.bias = (int32_t)b;
      if (op.requant_mode == TB200_REQUANT_NPU) {
        p.mult = mult[i] >> (shift[i] - min_shift);
        p.shift = min_shift;
      } else {
        p.mult = mult[i];
        p.shift = shift[i];
      }
      fill_rounding(p, double_round != 0);
      if (p.shift < 32) last_hi_shift = false;
      if (p.shift < last_min_shift) last_min_shift = p.shift;
      if (p.shift > last_max_shift) last_max_shift = p.shift;
      out[c] = p;
    }
    return true;
  }

  // set by chan_params: every shift of the op is >= 32 (the epilogue's one-word shift applies)
  bool last_hi_shift = true;
  int last_min_shift = 64;  // smallest effective shift of the op
  int last_max_shift = 0;   // largest

  // The compact "Q4" epilogue records {4 * bias, mult, rh, shift - 30} (common.cuh) for the channels in cp,
  // when the op qualifies: every shift in [32, 52], multipliers non-negative, and |4 * (acc + bias)| provably
  // below 2^31, where |acc| <= acc_bound[c] (from the weights: 128 * sum |w|, doubled when the kernel adds a
  // border correction). mode: 1 = with the sign term of DOUBLE_ROUND, 2 = without (single rounding, or the
  // clamp's lower end is at or above the output zero point so that every negative value lands on it anyway).
  // Returns 0 when the op does not qualify.
  static int q4_params(const std::vector<ChanParams>& cp, const std::vector<long long>& acc_bound, bool double_round,
                       int out_zp, int clamp_min, std::vector<int4>& out) {
    out.resize(cp.size());
    bool any_double = false;
    for (size_t c = 0; c < cp.size(); c++) {
      const ChanParams& p = cp[c];
      if (p.shift < 32 || p.shift > 52 || p.mult < 0) return 0;
      const long long b = p.bias;
      if ((acc_bound[c] + (b < 0 ? -b : b)) >= (1ll << 29)) return 0;
      const bool second = double_round && p.shift > 31;
      any_double |= second;
      const long long rh = (1ll << (p.shift - 31)) + ((long long)out_zp << (p.shift - 30)) + (second ? 1 : 0);
      // |mulhi(4v, M)| < 2^28 for |4v| < 2^31 and M < 2^31
      if (rh >= (1ll << 30) || rh <= -(1ll << 30)) return 0;
      out[c] = make_int4((int)(4 * b), p.mult, (int)rh, p.shift - 30);
    }
    return any_double && clamp_min < out_zp ? 1 : 2;
  }

  static void fill_rounding(ChanParams& p, bool double_round) {
    const bool second = double_round && p.shift > 31;
    p.rnd = (1ll << (p.shift - 1)) + (second ? (1ll << 30) : 0ll);
    p.dmul = second ? INT32_MIN : 0;
    p.hshift = p.shift - 32;
  }
};

// TOSA apply_scale_32 on the host (the device form is common.cuh's): value wrapped to int32 first, as the kernels do.
long long host_apply_scale_32(long long value, int mult, int shift, bool double_round) {
  const long long v = (long long)(int32_t)(uint32_t)(unsigned long long)value;
  long long round = 1ll << (shift - 1);
  if (double_round && shift > 31) round += v >= 0 ? (1ll << 30) : -(1ll << 30);
  return (long long)(int32_t)(uint32_t)(unsigned long long)((v * (long long)mult + round) >> shift);
}

// The parameters of a rescaled add / sub / mul without its pointers and size. The operand-side rescales are functions
// of one byte: both tables are evaluated here as the kernel does, the value that reaches the output rescale is
// bounded, and the 32-bit form of that rescale is taken when it is exact. False: a left shift outside [0, 22].
static bool binary_args_of(const tb200_op_t& op, BinaryArgs& a) {
  a = BinaryArgs{};
  a.kind = op.kind == TB200_OP_ADD ? 0 : op.kind == TB200_OP_SUB ? 1 : 2;
  a.a_zp = op.in0_zp; a.a_mult = op.in0_mult; a.a_shift = op.in0_shift;
  a.b_zp = op.in1_zp; a.b_mult = op.in1_mult; a.b_shift = op.in1_shift;
  a.out_mult = op.out_mult; a.out_shift = op.out_shift; a.out_zp = op.out_zp;
  a.double_round = op.double_round; a.clamp_min = op.clamp_min; a.clamp_max = op.clamp_max;
  if (op.i0 < 0 || op.i0 > 22 || op.i1 < 0 || op.i1 > 22) return false;
  for (int s : {op.in0_shift, op.in1_shift, op.out_shift})
    if (s < 2 || s > 62) return false;
  a.a_lshift = op.i0; a.b_lshift = op.i1;
  long long ma = 0, mb = 0;
  for (int v = -128; v < 128; v++) {
    const long long ra = host_apply_scale_32((long long)(v - a.a_zp) * (1ll << a.a_lshift), a.a_mult, a.a_shift, op.double_round != 0);
    const long long rb = host_apply_scale_32((long long)(v - a.b_zp) * (1ll << a.b_lshift), a.b_mult, a.b_shift, op.double_round != 0);
    ma = std::max(ma, ra < 0 ? -ra : ra);
    mb = std::max(mb, rb < 0 ? -rb : rb);
  }
  const long long bound = a.kind == 2 ? ma * mb : ma + mb;
  ChanParams cp{};
  cp.mult = a.out_mult; cp.shift = a.out_shift; cp.bias = 0;
  std::vector<int4> q4;
  a.epi = (ma < (1ll << 31) && mb < (1ll << 31) && bound < (1ll << 29))
              ? Builder::q4_params({cp}, {bound}, op.double_round != 0, a.out_zp, a.clamp_min, q4) : 0;
  if (a.epi) a.q4 = q4[0];
  return true;
}

int conv_out_dim(int i, int k, int s, int d, int p0, int p1) { return (i + p0 + p1 - d * (k - 1) - 1) / s + 1; }

bool force_simt() {
  const char* e = getenv("TB200_FORCE_SIMT");
  return e && *e && *e != '0';
}


// Rows of a 1x1 convolution / FullyConnected product that are read as one row against block-diagonal weights
// (row m' of the product then holds the outputs of pixels r*m' .. r*m'+r-1 back to back, which is exactly their dense
// NHWC placement, so nothing else changes).
static int pointwise_row_group(long long M, long long K, int OC) {
  // TMA wants a row pitch that is a multiple of 16 bytes
  int rgroup = 1;
  if (K % 16 != 0) {
    int g16 = 16;
    while (K % g16 != 0) g16 >>= 1;  // gcd(K, 16)
    rgroup = 16 / g16;
  }
  // Short rows make poor TMA boxes (the copy engine works row by row): widen them the same way while the grouped
  // row stays within one 128-byte swizzle row.
  while (rgroup * 2 <= 8 && K * rgroup * 2 <= 128 && M % (rgroup * 2) == 0 && OC * rgroup * 2 <= 512) rgroup *= 2;
  // An output row pitch that is no multiple of 16 bytes (24 channels) would leave the tile through byte stores
  // from registers (measured: 56x56 x 96 -> 24 at batch 256 took 88 us, 2 us per tile); grouped rows make the
  // pitch r * OC and the tile leaves as one TMA store. The block-diagonal weights multiply the tensor-core work
  // by r, which costs nothing here.
  while ((OC * rgroup) % 16 != 0 && rgroup * 2 <= 8 && M % (rgroup * 2) == 0 && OC * rgroup * 2 <= 512 &&
         K * rgroup * 2 <= 2048)
    rgroup *= 2;
  return rgroup;
}
// Whether that product runs on the tcgen05 GEMM (the few-row kernel and the CUDA-core convolution take the rest).
static bool pointwise_takes_gemm_tc(long long M, long long K, int OC, int weight_zp) {
  if (weight_zp != 0 || force_simt()) return false;
  if (M <= 4 && K % 16 == 0 && K <= 12288) return false;  // fc_rows_dp4a
  const int r = pointwise_row_group(M, K, OC);
  return r <= 8 && M % r == 0 && (long long)OC * r <= 65536 && gemm_tc_supported(M / r, OC * r, (int)K * r, K * r);
}

bool decode_per_op() {
  const char* e = getenv("TB200_DECODE_PER_OP");
  return e && *e && *e != '0';
}

// Recognises the whole-graph shape of one decode step (embed; per layer rmsnorm, gemv,
// rope_kv, attn_decode, gemv, rmsnorm+residual, rmsnorm, gemv, geglu, gemv, rmsnorm+residual;
// final rmsnorm, gemv to fp32 logits, argmax) and replaces its per-op launches by the one
// persistent kernel of decode_step.cu. Anything that does not fit exactly keeps the per-op plan.
bool try_fuse_decode_step(Builder& b, Plan& plan, size_t& scratch_need) {
  const auto& ops = b.ops;
  const auto& T = b.tensors;
  const int n = (int)ops.size();
  if (decode_per_op() || n < 15) return false;
  // Tensor-parallel shards carry an all-reduce after the o and the down projection.
  const bool tp_graph = ops[6].kind == TB200_OP_ALLREDUCE;
  const int stride = tp_graph ? 13 : 11;
  if ((n - 4) % stride != 0) return false;
  const int L = (n - 4) / stride;
  static const uint32_t layer_kinds[11] = {TB200_OP_RMSNORM, TB200_OP_GEMV_W8, TB200_OP_ROPE_KV, TB200_OP_ATTN_DECODE,
                                           TB200_OP_GEMV_W8, TB200_OP_RMSNORM, TB200_OP_RMSNORM, TB200_OP_GEMV_W8,
                                           TB200_OP_GEGLU,   TB200_OP_GEMV_W8, TB200_OP_RMSNORM};
  if (ops[0].kind != TB200_OP_EMBED || ops[n - 3].kind != TB200_OP_RMSNORM || ops[n - 2].kind != TB200_OP_GEMV_W8 ||
      ops[n - 1].kind != TB200_OP_ARGMAX)
    return false;
  // per layer: the 11 ops of the single-GPU form, and the two all-reduces when present
  std::vector<const tb200_op_t*> lo((size_t)L * 11), ar((size_t)L * 2, nullptr);
  for (int l = 0; l < L; l++) {
    int k = 0;
    for (int j = 0; j < stride; j++) {
      const tb200_op_t* op = &ops[1 + stride * l + j];
      if (tp_graph && (j == 5 || j == 11)) {
        if (op->kind != TB200_OP_ALLREDUCE) return false;
        ar[2 * l + (j == 11)] = op;
        continue;
      }
      if (op->kind != layer_kinds[k]) return false;
      lo[(size_t)11 * l + k++] = op;
    }
  }
  const int tp = tp_graph ? ar[0]->i0 : 1, rank = tp_graph ? ar[0]->i1 : 0;
  if (tp < 1 || tp > 8 || rank < 0 || rank >= tp) return false;
  auto inter = [&](int id) { return id >= 0 && T[id].kind == TB200_TENSOR_ACTIVATION; };
  const tb200_op_t& emb = ops[0];
  const int tokens = emb.in0;
  const int B = T[emb.in0].shape[0], V_embed = T[emb.weights].shape[0], H = T[emb.weights].shape[1];
  const int V = T[ops[n - 2].weights].shape[0];  // rows of this GPU's LM-head shard
  const tb200_op_t& first_rope = *lo[2];
  const int n_q = first_rope.i0, n_kv = first_rope.i1, D = first_rope.i2, pos = first_rope.in1;
  const int I = T[lo[8]->out0].shape[1];
  const int Tlen = T[first_rope.out1].shape[1];
  const float eps = lo[0]->f0, attn_scale = lo[3]->f0;
  if (!decode_step_supported(B, H, n_q, n_kv, D, I, V)) return false;
  // Measured on the 1B shape: the fused step wins at 1 and 2 sequences (1.17 ms against 1.43 ms at 2); from 3 on
  // the per-op path with the tensor-core GEMV is faster (1.44 ms against 1.57 ms at 3, 1.44 against 1.70 at 4,
  // 1.47 against 2.83 at 8). Tensor-parallel shards exist only in fused form. TB200_DECODE_FUSED_MAX_B moves
  // the threshold.
  {
    const char* e = getenv("TB200_DECODE_FUSED_MAX_B");
    const int max_b = e ? atoi(e) : 2;
    if (!tp_graph && B > max_b) return false;
  }
  int dev = 0, sms = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
    return false;
  // every CTA must own at least one row of every projection (the barrier protocol counts on it)
  if (sms < 1 || H < sms || I < sms || V < sms || (n_q + 2) * D < sms) return false;
  if (T[tokens].kind != TB200_TENSOR_INPUT || T[pos].kind != TB200_TENSOR_INPUT) return false;

  std::vector<DecodeLayerDesc> descs(L);
  float thetas[2] = {0.f, 0.f};
  size_t off = 0;
  auto cst = [&](int id, size_t bytes, unsigned long long& dst) {
    if (!b.add_raw_const(id, bytes, "decode-step constant", 0, off)) return false;
    dst = off;
    return true;
  };
  auto gemv_ok = [&](const tb200_op_t& g, int in, int N, int K, bool f32) {
    return g.in0 == in && inter(in) && T[g.weights].rank == 2 && T[g.weights].shape[0] == N && T[g.weights].shape[1] == K &&
           T[g.out0].dtype == (f32 ? TB200_F32 : TB200_BF16) && T[g.in0].shape[0] == B && g.i1 == 0 &&
           T[g.in0].shape[1] == K;
  };
  // the o projection may take a K slice of the attention output (a head shared by two GPUs)
  const int o_k = T[lo[4]->weights].shape[1], o_k_offset = lo[4]->i1;
  if (o_k < 64 || o_k % 64 != 0 || o_k_offset < 0 || o_k_offset % 8 != 0 || o_k_offset + o_k > n_q * D) return false;
  if (!tp_graph && (o_k != n_q * D || o_k_offset != 0)) return false;
  auto norm_ok = [&](const tb200_op_t& r, int in, int res) {
    return r.in0 == in && r.in1 == res && r.f0 == eps && T[r.in0].shape[1] == H && T[r.in0].shape[0] == B;
  };
  int x = emb.out0;
  if (!inter(x)) return false;
  for (int l = 0; l < L; l++) {
    tb200_op_t o[11];
    for (int k = 0; k < 11; k++) o[k] = *lo[(size_t)11 * l + k];
    DecodeLayerDesc& d = descs[l];
    if (!norm_ok(o[0], x, -1) || !gemv_ok(o[1], o[0].out0, (n_q + 2) * D, H, false)) return false;
    const tb200_op_t& rope = o[2];
    const tb200_op_t& att = o[3];
    if (rope.in0 != o[1].out0 || !inter(rope.in0) || rope.in1 != pos || rope.i0 != n_q || rope.i1 != n_kv || rope.i2 != D ||
        rope.f1 != eps || T[rope.out1].shape[1] != Tlen || !inter(rope.out0))
      return false;
    if (att.in0 != rope.out0 || att.in1 != pos || att.in2 != rope.out1 || att.weights != rope.in2 || att.i0 != n_q ||
        att.i1 != n_kv || att.i2 != D || att.f0 != attn_scale || att.i3 < 0)
      return false;
    // with tensor parallelism the K-split projections give fp32 partial results, summed by the all-reduce
    auto reduced = [&](const tb200_op_t& g, const tb200_op_t* red) {
      if (!tp_graph) return g.out0;
      if (!red || red->in0 != g.out0 || !inter(g.out0) || red->i0 != tp || red->i1 != rank || T[red->in0].dtype != TB200_F32 ||
          T[red->out0].dtype != TB200_BF16 || b.numel(red->in0) != b.numel(red->out0))
        return -1;
      return red->out0;
    };
    const int o_out = reduced(o[4], ar[2 * l]);
    {
      const tb200_op_t& og = o[4];  // like gemv_ok, with the K slice
      if (og.in0 != att.out0 || !inter(og.in0) || T[og.weights].rank != 2 || T[og.weights].shape[0] != H ||
          T[og.weights].shape[1] != o_k || og.i1 != o_k_offset || T[og.out0].dtype != (tp_graph ? TB200_F32 : TB200_BF16))
        return false;
    }
    if (o_out < 0 || !norm_ok(o[5], o_out, x) || !inter(o_out)) return false;
    x = o[5].out0;
    if (!inter(x) || !norm_ok(o[6], x, -1) || !gemv_ok(o[7], o[6].out0, 2 * I, H, false)) return false;
    if (o[8].in0 != o[7].out0 || !inter(o[8].in0) || T[o[8].out0].shape[1] != I) return false;
    const int d_out = reduced(o[9], ar[2 * l + 1]);
    if (d_out < 0 || !gemv_ok(o[9], o[8].out0, H, I, tp_graph) || !norm_ok(o[10], d_out, x) || !inter(d_out)) return false;
    x = o[10].out0;
    if (!inter(x)) return false;
    if (!cst(o[0].weights, (size_t)H * 2, d.in_norm) || !cst(o[1].weights, (size_t)(n_q + 2) * D * H, d.w_qkv) ||
        !cst(o[1].bias, (size_t)(n_q + 2) * D * 2, d.s_qkv) || !cst(rope.weights, (size_t)D * 2, d.q_norm) ||
        !cst(rope.bias, (size_t)D * 2, d.k_norm) || !cst(o[4].weights, (size_t)H * o_k, d.w_o) ||
        !cst(o[4].bias, (size_t)H * 2, d.s_o) || !cst(o[5].weights, (size_t)H * 2, d.post_attn_norm) ||
        !cst(o[6].weights, (size_t)H * 2, d.pre_ffn_norm) || !cst(o[7].weights, (size_t)2 * I * H, d.w_gu) ||
        !cst(o[7].bias, (size_t)2 * I * 2, d.s_gu) || !cst(o[9].weights, (size_t)H * I, d.w_down) ||
        !cst(o[9].bias, (size_t)H * 2, d.s_down) || !cst(o[10].weights, (size_t)H * 2, d.post_ffn_norm))
      return false;
    d.kcache = plan.tensor_loc[rope.out1].offset;
    d.vcache = plan.tensor_loc[rope.in2].offset;
    d.theta = rope.f0;
    d.window = att.i3;
    // at most two RoPE bases (local and global layers) share the kernel's two tables
    if (l == 0) thetas[0] = thetas[1] = rope.f0;
    if (rope.f0 == thetas[0]) d.rope_table = 0;
    else if (thetas[1] == thetas[0] || rope.f0 == thetas[1]) { thetas[1] = rope.f0; d.rope_table = 1; }
    else return false;
    // the fp16 copy of a normed vector is exact only while |1 + w| stays moderate
    for (int id : {o[0].weights, o[5].weights, o[6].weights, o[10].weights}) {
      const uint16_t* w = b.const_data<uint16_t>(id, H, "norm weight", 0);
      if (!w) return false;
      for (int i = 0; i < H; i++) {
        const uint32_t bits = (uint32_t)w[i] << 16;
        float f;
        memcpy(&f, &bits, 4);
        if (!(f > -257.0f && f < 255.0f)) return false;
      }
    }
  }
  const tb200_op_t& nf = ops[n - 3];
  const tb200_op_t& lm = ops[n - 2];
  const tb200_op_t& am = ops[n - 1];
  if (!norm_ok(nf, x, -1) || !gemv_ok(lm, nf.out0, V, H, true) || am.in0 != lm.out0 ||
      T[am.out0].kind != TB200_TENSOR_OUTPUT || T[am.out0].shape[0] != B)
    return false;
  if (!tp_graph && (lm.weights != emb.weights || lm.bias != emb.bias || am.i1 > 1)) return false;
  if (tp_graph && (am.i1 != tp || am.i0 < 0)) return false;  // arg max over every GPU's shard, ids offset by i0
  const bool logits_out = T[lm.out0].kind == TB200_TENSOR_OUTPUT;
  if (!logits_out && !inter(lm.out0)) return false;

  DecodeStepArgs a{};
  if (!cst(emb.weights, (size_t)V_embed * H, a.embed_w) || !cst(emb.bias, (size_t)V_embed * 2, a.embed_s) ||
      !cst(lm.weights, (size_t)V * H, a.lm_w) || !cst(lm.bias, (size_t)V * 2, a.lm_s) ||
      !cst(nf.weights, (size_t)H * 2, a.final_norm))
    return false;
  a.layers_off = b.add_const(descs.data(), descs.size() * sizeof(DecodeLayerDesc));
  a.n_layers = L; a.B = B; a.H = H; a.n_q = n_q; a.I = I; a.V = V; a.V_embed = V_embed; a.T = Tlen;
  a.tp = tp; a.rank = rank; a.vocab_offset = tp_graph ? am.i0 : 0;
  a.o_k = o_k; a.o_k_offset = o_k_offset;
  a.eps = eps; a.attn_scale = attn_scale; a.embed_mult = emb.f0; a.grid = sms;
  a.theta[0] = thetas[0]; a.theta[1] = thetas[1];
  scratch_need = std::max(scratch_need, decode_step_scratch_bytes(B, H, n_q, I, L, sms, tp, &a));
  const Loc ltok = plan.tensor_loc[tokens], lpos = plan.tensor_loc[pos], lids = plan.tensor_loc[am.out0],
            llog = plan.tensor_loc[lm.out0];
  for (auto& st : plan.steps) {
    st.kernel_name = "(in decode_step)";
    st.launches = 0;
    st.launch = [](const ExecContext&) {};
  }
  plan.steps[0].kernel_name = "decode_step_persistent";
  plan.steps[0].launches = 1;
  // TB200_DECODE_TRACE=<file>: after every dispatch, wait for it and append CTA 0's stage
  // timestamps (ns, one line per dispatch) to the file. For profiling only: it serialises.
  const char* trace_env = getenv("TB200_DECODE_TRACE");
  const std::string trace_path = trace_env ? trace_env : "";
  if (trace_path.empty()) a.trace_off = 0;
  plan.steps[0].launch = [=](const ExecContext& c) {
    DecodeStepArgs k = a;
    k.consts = c.consts; k.arena = c.arena; k.scratch = c.scratch; k.status = c.status;
    for (int r = 0; r < 8; r++) k.peer_scratch[r] = nullptr;
    k.peer_scratch[rank] = c.scratch;
    if (tp > 1) {
      if (!c.peer_scratch) {
        if (c.launch_error) *c.launch_error = cudaErrorNotReady;  // the peers have not been connected yet
        return;
      }
      for (int r = 0; r < tp; r++) k.peer_scratch[r] = c.peer_scratch[r];
    }
    k.tokens = (const int32_t*)ltok.resolve(c);
    k.pos = (const int32_t*)lpos.resolve(c);
    k.out_ids = (int32_t*)lids.resolve(c);
    k.logits = logits_out ? (float*)llog.resolve(c) : nullptr;
    const cudaError_t e = launch_decode_step(k, c.stream);
    if (e != cudaSuccess && c.launch_error) *c.launch_error = e;
    if (e == cudaSuccess && !trace_path.empty() && cudaStreamSynchronize(c.stream) == cudaSuccess) {
      std::vector<unsigned long long> t(k.trace_len);
      if (cudaMemcpy(t.data(), c.scratch + k.trace_off, t.size() * 8, cudaMemcpyDeviceToHost) == cudaSuccess) {
        if (FILE* f = fopen(trace_path.c_str(), "a")) {
          for (size_t i = 0; i < t.size(); i++) fprintf(f, "%llu%c", t[i] - t[0], i + 1 < t.size() ? ',' : '\n');
          fclose(f);
        }
      }
    }
  };
  plan.launch_count = 1;
  plan.use_graph = false;    // one launch per dispatch: nothing for a graph to save
  plan.tp = tp;
  plan.rank = rank;
  plan.zero_scratch = true;  // the grid-barrier counters start at zero
  return true;
}

}  // namespace

int build_plan(const std::vector<tb200_tensor_t>& tensors, const std::vector<tb200_op_t>& ops,
               const std::vector<uint8_t>& constants, Plan& plan, std::string& err) {
  Builder b{tensors, ops, constants, plan, err};
  const int nt = (int)tensors.size();

  // ---- tensor placement: io slots, state prefix, liveness-packed activations ----
  plan.tensor_loc.assign(nt, Loc{});
  std::vector<int> first_def(nt, -1), last_use(nt, -1), root(nt);
  for (int id = 0; id < nt; id++) root[id] = id;
  // Chained concats: concat(concat(p, q), r) where the inner result is used nowhere else and the
  // outer op passes it through unchanged (multiplier 2^30, shift 30, equal zero points) is written in
  // place: the inner result becomes the leading columns of the outer one (same storage, the outer
  // row stride) and the outer op only adds its second operand.
  std::vector<int> concat_into(nt, -1);  // inner result tensor -> outer result tensor
  // A 256-entry table that is the only reader of a convolution's result (the reference fuses the same
  // pair: OptimizeSwishActivationPattern.cpp:100-190) is applied in the convolution's epilogue.
  std::vector<int> table_after(ops.size(), -1);  // conv op -> index of its fused table op
  std::vector<char> fused_away(ops.size(), 0);
  std::vector<int> add_after(ops.size(), -1);      // conv op -> index of the add fused into its epilogue
  std::vector<char> add_self_is_a(ops.size(), 0);  // the convolution's result is the add's first operand
  // Decoder graphs run op by op: (1) a split-K gemv_w8 whose only reader is the next op (rmsnorm, rope_kv or
  // geglu) leaves its per-slice sums in scratch and the reader finalizes them as it loads; (2) an rmsnorm
  // directly followed by an rmsnorm of its result runs as one launch. Same arithmetic, fewer launches.
  std::vector<int> partials_from(ops.size(), -1);  // reader op -> the gemv_w8 op whose partial sums it takes
  std::vector<char> defer_finalize(ops.size(), 0);
  std::vector<int> norm_second(ops.size(), -1);    // rmsnorm op -> the rmsnorm op fused into it
  std::vector<int> extra_out(ops.size(), -1);      // tensor an op writes on behalf of the op fused into it
  {
    std::vector<int> uses(nt, 0), producer(nt, -1);
    for (int i = 0; i < (int)ops.size(); i++) {
      for (int id : {ops[i].in0, ops[i].in1, ops[i].in2, ops[i].weights})
        if (id >= 0 && id < nt) uses[id]++;
      for (int id : {ops[i].out0, ops[i].out1})
        if (id >= 0 && id < nt) producer[id] = i;
    }
    for (int i = 0; i < (int)ops.size(); i++) {
      const auto& op = ops[i];
      if (op.kind != TB200_OP_CONCAT || op.in0 < 0 || op.in0 >= nt || op.out0 < 0 || op.out0 >= nt) continue;
      const int a = op.in0, pa = producer[a];
      if (pa < 0 || ops[pa].kind != TB200_OP_CONCAT || uses[a] != 1 || tensors[a].kind != TB200_TENSOR_ACTIVATION ||
          tensors[op.out0].kind != TB200_TENSOR_ACTIVATION)
        continue;
      if (op.in0_mult == (1 << 30) && op.in0_shift == 30 && op.in0_zp == op.out_zp && tensors[a].dtype == TB200_I8)
        concat_into[a] = op.out0;
    }
    const char* no_fuse = getenv("TB200_NO_TABLE_FUSION");
    for (int i = 0; i < (int)ops.size() && !(no_fuse && *no_fuse && *no_fuse != '0'); i++) {
      const auto& op = ops[i];
      if (op.kind != TB200_OP_TABLE || op.in0 < 0 || op.in0 >= nt || op.out0 < 0 || op.out0 >= nt) continue;
      const int src = op.in0, pc = producer[src];
      if (pc < 0 || pc >= i || ops[pc].kind != TB200_OP_CONV2D || uses[src] != 1 || table_after[pc] >= 0 ||
          tensors[src].kind != TB200_TENSOR_ACTIVATION || tensors[src].dtype != TB200_I8 || tensors[op.out0].dtype != TB200_I8)
        continue;
      table_after[pc] = i;
      fused_away[i] = 1;
      extra_out[pc] = op.out0;
    }
    // A rescaled add whose one operand is the only use of a 1x1 convolution's result (a residual connection) runs
    // in that convolution's epilogue when the convolution takes the tensor-core GEMM: the other operand is read
    // there, the product never goes to memory. The add's own checks (and its 32-bit output rescale, which the
    // fused form requires) happen when the convolution is planned; what cannot be fused there fails the plan
    // no differently from the stand-alone op.
    // Off unless TB200_ADD_FUSION=1: measured on MobileNetV2 at batch 256 the fused form is no faster (1.693 ms per
    // step against 1.678 with the ten adds as their own launches) - the step is bound by integer issue slots, and the
    // add's table look-ups, rescale and repacking cost the same slots wherever they run.
    const char* do_add = getenv("TB200_ADD_FUSION");
    for (int i = 0; i < (int)ops.size() && do_add && *do_add && *do_add != '0'; i++) {
      const auto& op = ops[i];
      if (op.kind != TB200_OP_ADD || op.in0 < 0 || op.in0 >= nt || op.in1 < 0 || op.in1 >= nt || op.out0 < 0 || op.out0 >= nt ||
          op.in0 == op.in1)
        continue;
      for (int side = 0; side < 2; side++) {
        const int src = side == 0 ? op.in0 : op.in1, other = side == 0 ? op.in1 : op.in0;
        const int pc = producer[src];
        if (pc < 0 || pc >= i || ops[pc].kind != TB200_OP_CONV2D || uses[src] != 1 || table_after[pc] >= 0 || add_after[pc] >= 0 ||
            tensors[src].kind != TB200_TENSOR_ACTIVATION || tensors[src].dtype != TB200_I8 || tensors[op.out0].dtype != TB200_I8 ||
            tensors[other].dtype != TB200_I8 || tensors[other].kind == TB200_TENSOR_CONSTANT)
          continue;
        // the other operand must exist when the convolution runs
        if (tensors[other].kind != TB200_TENSOR_INPUT && (producer[other] < 0 || producer[other] >= pc)) continue;
        const auto& cv = ops[pc];
        if (cv.in0 < 0 || cv.in0 >= nt || cv.weights < 0 || cv.weights >= nt || tensors[cv.in0].rank != 4 ||
            tensors[cv.weights].rank != 4 || tensors[src].rank != 4)
          continue;
        const auto& x = tensors[cv.in0]; const auto& w = tensors[cv.weights]; const auto& o = tensors[src];
        if (w.shape[1] != 1 || w.shape[2] != 1 || cv.stride_h != 1 || cv.stride_w != 1 || cv.pad_t || cv.pad_b || cv.pad_l || cv.pad_r)
          continue;
        const long long M = (long long)x.shape[0] * x.shape[1] * x.shape[2];
        const int OC = w.shape[0];
        if (!pointwise_takes_gemm_tc(M, x.shape[3], OC, cv.weight_zp)) continue;
        if ((long long)o.shape[0] * o.shape[1] * o.shape[2] != M || o.shape[3] != OC) continue;
        bool same = tensors[other].rank == 4 && tensors[op.out0].rank == 4;
        for (int d = 0; d < 4 && same; d++) same = tensors[other].shape[d] == o.shape[d] && tensors[op.out0].shape[d] == o.shape[d];
        if (!same) continue;
        // the fused form exists for the 32-bit output rescale only
        BinaryArgs probe{};
        if (!binary_args_of(op, probe) || probe.epi == 0) continue;
        add_after[pc] = i;
        add_self_is_a[pc] = side == 0;
        fused_away[i] = 1;
        extra_out[pc] = op.out0;
        break;
      }
    }
    const char* no_dec = getenv("TB200_NO_DECODER_FUSION");
    for (int i = 0; i + 1 < (int)ops.size() && !(no_dec && *no_dec && *no_dec != '0'); i++) {
      const auto& op = ops[i];
      const auto& nx = ops[i + 1];
      auto ok2d = [&](int id, int dtype) {
        return id >= 0 && id < nt && tensors[id].rank == 2 && tensors[id].dtype == dtype;
      };
      if (op.kind == TB200_OP_GEMV_W8 && ok2d(op.in0, TB200_BF16) && ok2d(op.out0, TB200_BF16) && ok2d(op.weights, TB200_I8) &&
          tensors[op.out0].kind == TB200_TENSOR_ACTIVATION && uses[op.out0] == 1 && nx.in0 == op.out0 && op.i1 == 0 &&
          (nx.kind == TB200_OP_RMSNORM || nx.kind == TB200_OP_ROPE_KV || nx.kind == TB200_OP_GEGLU)) {
        const int B = tensors[op.in0].shape[0], N = tensors[op.weights].shape[0], K = tensors[op.weights].shape[1];
        const bool plain = K == tensors[op.in0].shape[1] && K > 0 && K % 16 == 0 && B >= 1 && B <= 32 && N >= 1;
        if (plain && !(nx.kind == TB200_OP_RMSNORM && N > 8192)) {
          const int splits = op.i0 > 0 ? op.i0 : gemv_w8_splits(B, N, K);
          if (gemv_w8_used_splits(B, N, K, splits) > 1) {
            defer_finalize[i] = 1;
            partials_from[i + 1] = i;
          }
        }
      }
      if (op.kind == TB200_OP_RMSNORM && nx.kind == TB200_OP_RMSNORM && !fused_away[i] && nx.in0 == op.out0 && nx.in1 < 0 &&
          ok2d(op.in0, TB200_BF16) && ok2d(op.out0, TB200_BF16) && ok2d(nx.out0, TB200_BF16) && nx.out0 != op.out0 &&
          tensors[op.in0].shape[1] <= 8192 && tensors[nx.out0].shape[0] == tensors[op.out0].shape[0] &&
          tensors[nx.out0].shape[1] == tensors[op.out0].shape[1] && tensors[op.out0].shape[1] == tensors[op.in0].shape[1] &&
          tensors[op.out0].shape[0] == tensors[op.in0].shape[0]) {
        norm_second[i] = i + 1;
        fused_away[i + 1] = 1;
        extra_out[i] = nx.out0;
      }
    }
  }
  for (int i = 0; i < (int)ops.size(); i++) {
    const auto& op = ops[i];
    int ins[3] = {op.in0, op.in1, op.in2};
    int outs[3] = {op.out0, op.out1, extra_out[i]};
    for (int id : ins)
      if (id >= 0) {
        if (!b.valid_id(id)) return b.fail(TB200_INVALID_ARGUMENT, "op %d: input tensor id %d out of range", i, id);
        last_use[root[id]] = i;
      }
    for (int id : outs)
      if (id >= 0) {
        if (!b.valid_id(id)) return b.fail(TB200_INVALID_ARGUMENT, "op %d: output tensor id %d out of range", i, id);
        if (tensors[id].kind == TB200_TENSOR_CONSTANT || tensors[id].kind == TB200_TENSOR_INPUT)
          return b.fail(TB200_INVALID_ARGUMENT, "op %d writes tensor %d which is not writable", i, id);
        if (first_def[id] < 0) first_def[id] = i;
        last_use[id] = std::max(last_use[id], i);
      }
    if (op.kind == TB200_OP_CONCAT && op.out0 >= 0 && concat_into[op.out0] >= 0) {
      // written in place into the outer concat's result: that tensor's storage starts living here
      int fin = op.out0;
      while (concat_into[fin] >= 0) fin = concat_into[fin];
      root[op.out0] = fin;
      if (first_def[fin] < 0 || first_def[fin] > i) first_def[fin] = i;
      last_use[fin] = std::max(last_use[fin], i);
    }
    if (op.kind == TB200_OP_RESHAPE) {
      // a view: shares the storage (and the lifetime) of what it reshapes
      if (op.in0 < 0 || op.out0 < 0 || tensors[op.in0].kind == TB200_TENSOR_CONSTANT ||
          (tensors[op.out0].kind != TB200_TENSOR_ACTIVATION && tensors[op.out0].kind != TB200_TENSOR_OUTPUT))
        return b.fail(TB200_INVALID_ARGUMENT, "op %d: reshape wants a non-constant input and a writable result", i);
      // a reshape that produces a graph output cannot alias (the output has its own binding): it copies
      if (tensors[op.out0].kind == TB200_TENSOR_ACTIVATION) root[op.out0] = root[op.in0];
    }
  }
  auto bytes_of = [&](int id) {
    size_t n = b.numel(id);
    switch (tensors[id].dtype) {
      case TB200_I8: return n;
      case TB200_I16: case TB200_BF16: return n * 2;
      case TB200_I64: return n * 8;
      default: return n * 4;
    }
  };
  size_t cursor = 0;
  for (int id = 0; id < nt; id++)
    if (tensors[id].kind == TB200_TENSOR_STATE) {
      plan.tensor_loc[id] = Loc{Loc::ARENA, cursor};
      cursor += (bytes_of(id) + 255) & ~(size_t)255;
    }
  plan.state_bytes = cursor;
  {
    struct Block { size_t off, size; int id; };
    std::vector<Block> live;
    size_t high = cursor;
    const size_t base = cursor;
    for (int i = 0; i < (int)ops.size(); i++) {
      int outs[3] = {ops[i].out0, ops[i].out1, extra_out[i]};
      for (int out_id : outs) {
        // a result written in place into a later tensor (concat chains) allocates that tensor now
        const int id = out_id >= 0 && ops[i].kind == TB200_OP_CONCAT ? root[out_id] : out_id;
        if (id < 0 || tensors[id].kind != TB200_TENSOR_ACTIVATION || first_def[id] != i) continue;
        if (plan.tensor_loc[id].kind != Loc::NONE || root[id] != id) continue;
        size_t need = (bytes_of(id) + 255) & ~(size_t)255;
        std::sort(live.begin(), live.end(), [](const Block& x, const Block& y) { return x.off < y.off; });
        size_t pos = base;
        for (const auto& blk : live) {
          if (blk.off >= pos + need) break;
          pos = std::max(pos, blk.off + blk.size);
        }
        live.push_back({pos, need, id});
        plan.tensor_loc[id] = Loc{Loc::ARENA, pos};
        high = std::max(high, pos + need);
      }
      live.erase(std::remove_if(live.begin(), live.end(), [&](const Block& blk) { return last_use[blk.id] <= i; }),
                 live.end());
    }
    plan.arena_bytes = high;
  }
  {
    // io slots are assigned by the order of the blob's input/output lists, which the
    // caller of build_plan cannot see here; tensors carry their slot in `reserved`.
    for (int id = 0; id < nt; id++)
      if (tensors[id].kind == TB200_TENSOR_INPUT || tensors[id].kind == TB200_TENSOR_OUTPUT)
        plan.tensor_loc[id] = Loc{Loc::IO, tensors[id].reserved};
    for (int id = 0; id < nt; id++)
      if (root[id] != id) plan.tensor_loc[id] = plan.tensor_loc[root[id]];
  }

  size_t scratch_need = 0;
  struct DeferredGemv { size_t scale_off; int splits; };
  std::vector<DeferredGemv> deferred(ops.size(), DeferredGemv{0, 0});
  // the operand a reader of deferred partial sums passes to its kernel
  auto partials_of = [&](int reader) {
    const int src = partials_from[reader];
    return src >= 0 ? deferred[src] : DeferredGemv{0, 0};
  };
  bool needs_fusion = false;  // the graph holds ops that exist only inside the fused decode step
  // ---- one step per op ----
  for (int i = 0; i < (int)ops.size(); i++) {
    const auto& op = ops[i];
    Step step;
    // a constant tensor used as a runtime operand (the generic tensor ops) is uploaded as it is
    auto loc = [&](int id) {
      if (id < 0) return Loc{};
      if (tensors[id].kind == TB200_TENSOR_CONSTANT && plan.tensor_loc[id].kind == Loc::NONE) {
        size_t off = 0;
        if (b.add_raw_const(id, 0, "operand", i, off)) plan.tensor_loc[id] = Loc{Loc::CONST, off};
      }
      return plan.tensor_loc[id];
    };
    for (int id : {op.in0, op.in1, op.in2})
      if (id >= 0 && tensors[id].kind != TB200_TENSOR_CONSTANT && plan.tensor_loc[id].kind == Loc::NONE)
        return b.fail(TB200_INVALID_ARGUMENT, "op %d reads tensor %d before anything wrote it", i, id);

    if (fused_away[i]) {
      step.kernel_name = op.kind == TB200_OP_RMSNORM ? "(norm fused into the previous norm)"
                         : op.kind == TB200_OP_ADD   ? "(add in the convolution's epilogue)"
                                                     : "(table in the convolution's epilogue)";
      step.launches = 0;
      step.launch = [](const ExecContext&) {};
      plan.steps.push_back(std::move(step));
      continue;
    }
    switch (op.kind) {
      case TB200_OP_CONV2D_I16: {
        if (!b.valid_id(op.in0) || !b.valid_id(op.out0) || !b.valid_id(op.weights) || tensors[op.in0].dtype != TB200_I16 ||
            tensors[op.out0].dtype != TB200_I16 || tensors[op.in0].rank != 4 || tensors[op.out0].rank != 4 ||
            tensors[op.weights].rank != 4)
          return b.fail(TB200_INVALID_ARGUMENT, "op %d: conv2d_i16 wants int16 NHWC input/output and OHWI int8 weights", i);
        const auto& x = tensors[op.in0]; const auto& w = tensors[op.weights]; const auto& o = tensors[op.out0];
        ConvI16Args a{};
        a.N = x.shape[0]; a.H = x.shape[1]; a.W = x.shape[2]; a.IC = x.shape[3];
        a.OC = w.shape[0]; a.KH = w.shape[1]; a.KW = w.shape[2];
        if (w.shape[3] != a.IC) return b.fail(TB200_INVALID_ARGUMENT, "op %d: weight IC %d != input IC %d", i, w.shape[3], a.IC);
        if (op.stride_h < 1 || op.stride_w < 1 || op.dil_h < 1 || op.dil_w < 1 || op.pad_t < 0 || op.pad_b < 0 || op.pad_l < 0 ||
            op.pad_r < 0)
          return b.fail(TB200_INVALID_ARGUMENT, "op %d: bad stride/dilation/pad", i);
        a.OH = conv_out_dim(a.H, a.KH, op.stride_h, op.dil_h, op.pad_t, op.pad_b);
        a.OW = conv_out_dim(a.W, a.KW, op.stride_w, op.dil_w, op.pad_l, op.pad_r);
        if (o.shape[0] != a.N || o.shape[1] != a.OH || o.shape[2] != a.OW || o.shape[3] != a.OC)
          return b.fail(TB200_INVALID_ARGUMENT, "op %d: conv2d_i16 output shape is not %dx%dx%dx%d", i, a.N, a.OH, a.OW, a.OC);
        const size_t wn = (size_t)a.OC * a.KH * a.KW * a.IC;
        const int8_t* wd = b.const_data<int8_t>(op.weights, wn, "weights", i);
        if (!wd) return b.status;
        const int n_bias = b.valid_id(op.bias) ? (int)b.numel(op.bias) : 0, n_q = op.per_channel ? a.OC : 1;
        if (n_bias != 1 && n_bias != a.OC) return b.fail(TB200_INVALID_ARGUMENT, "op %d: bias wants 1 or OC int64 entries", i);
        const long long* bias = b.const_data<long long>(op.bias, (size_t)n_bias, "bias", i);
        const int32_t* mult = b.const_data<int32_t>(op.multiplier, (size_t)n_q, "multiplier", i);
        const int8_t* shift = b.const_data<int8_t>(op.shift, (size_t)n_q, "shift", i);
        if (!bias || !mult || !shift) return b.status;
        std::vector<long long> bias_v(a.OC);
        std::vector<int32_t> mult_v(a.OC), shift_v(a.OC);
        for (int oc = 0; oc < a.OC; oc++) {
          bias_v[oc] = bias[n_bias == 1 ? 0 : oc];
          mult_v[oc] = mult[op.per_channel ? oc : 0];
          shift_v[oc] = shift[op.per_channel ? oc : 0];
          if (mult_v[oc] < 0 || mult_v[oc] > 32767 || shift_v[oc] < 2 || shift_v[oc] > 62)
            return b.fail(TB200_INVALID_ARGUMENT, "op %d: 16-bit rescale wants 0 <= multiplier < 2^15 and 2 <= shift <= 62", i);
        }
        const size_t w_off = b.add_const(wd, wn), b_off = b.add_const(bias_v.data(), bias_v.size() * 8),
                     m_off = b.add_const(mult_v.data(), mult_v.size() * 4), s_off = b.add_const(shift_v.data(), shift_v.size() * 4);
        a.stride_h = op.stride_h; a.stride_w = op.stride_w; a.dil_h = op.dil_h; a.dil_w = op.dil_w;
        a.pad_t = op.pad_t; a.pad_l = op.pad_l;
        a.input_zp = op.in0_zp; a.weight_zp = op.weight_zp; a.out_zp = op.out_zp;
        a.clamp_min = op.clamp_min < -32768 ? -32768 : op.clamp_min;
        a.clamp_max = op.clamp_max > 32767 ? 32767 : op.clamp_max;
        Loc lx = loc(op.in0), lo = loc(op.out0);
        step.kernel_name = "conv2d_i16";
        step.launch = [=](const ExecContext& c) {
          ConvI16Args k = a;
          k.x = (const int16_t*)lx.resolve(c);
          k.out = (int16_t*)lo.resolve(c);
          k.w = (const int8_t*)(c.consts + w_off);
          k.bias = (const long long*)(c.consts + b_off);
          k.mult = (const int32_t*)(c.consts + m_off);
          k.shift = (const int32_t*)(c.consts + s_off);
          launch_conv2d_i16(k, c.stream);
        };
        break;
      }
      case TB200_OP_CONV2D:
      case TB200_OP_FC: {
        const bool fc = op.kind == TB200_OP_FC;
        // a table fused into the epilogue: the result goes to the table op's output
        const int fused_table = table_after[i];
        const int result_id = fused_table >= 0 ? ops[fused_table].out0 : op.out0;
        size_t lut_off = 0;
        if (fused_table >= 0) {
          const int8_t* tbl = b.const_data<int8_t>(ops[fused_table].table, 256, "table", fused_table);
          if (!tbl) return b.status;
          if (b.numel(ops[fused_table].out0) != b.numel(op.out0))
            return b.fail(TB200_INVALID_ARGUMENT, "op %d: table wants int8 input/output of equal size", fused_table);
          lut_off = b.add_const(tbl, 256);
        }
        const bool has_lut = fused_table >= 0;
        int N, H, W, IC, OC, KH, KW, OH, OW;
        if (fc) {
          if (!b.act_i8(op.in0, 2) || !b.act_i8(op.out0, 2) || !b.valid_id(op.weights) || tensors[op.weights].rank != 2)
            return b.fail(TB200_INVALID_ARGUMENT, "op %d: fully_connected wants int8 [M,K] x [N,K] -> [M,N]", i);
          N = tensors[op.in0].shape[0]; H = W = 1; IC = tensors[op.in0].shape[1];
          OC = tensors[op.weights].shape[0]; KH = KW = 1; OH = OW = 1;
          if (tensors[op.weights].shape[1] != IC || tensors[op.out0].shape[0] != N || tensors[op.out0].shape[1] != OC)
            return b.fail(TB200_INVALID_ARGUMENT, "op %d: fully_connected shape mismatch", i);
        } else {
          if (!b.act_i8(op.in0, 4) || !b.act_i8(op.out0, 4) || !b.valid_id(op.weights) || tensors[op.weights].rank != 4)
            return b.fail(TB200_INVALID_ARGUMENT, "op %d: conv2d wants int8 NHWC input/output and OHWI weights", i);
          const auto& x = tensors[op.in0]; const auto& w = tensors[op.weights]; const auto& o = tensors[op.out0];
          N = x.shape[0]; H = x.shape[1]; W = x.shape[2]; IC = x.shape[3];
          OC = w.shape[0]; KH = w.shape[1]; KW = w.shape[2];
          if (w.shape[3] != IC) return b.fail(TB200_INVALID_ARGUMENT, "op %d: weight IC %d != input IC %d", i, w.shape[3], IC);
          if (op.stride_h < 1 || op.stride_w < 1 || op.dil_h < 1 || op.dil_w < 1 || op.pad_t < 0 || op.pad_b < 0 ||
              op.pad_l < 0 || op.pad_r < 0)
            return b.fail(TB200_INVALID_ARGUMENT, "op %d: bad stride/dilation/pad", i);
          OH = conv_out_dim(H, KH, op.stride_h, op.dil_h, op.pad_t, op.pad_b);
          OW = conv_out_dim(W, KW, op.stride_w, op.dil_w, op.pad_l, op.pad_r);
          if (o.shape[0] != N || o.shape[1] != OH || o.shape[2] != OW || o.shape[3] != OC)
            return b.fail(TB200_INVALID_ARGUMENT, "op %d: conv2d output shape is not %dx%dx%dx%d", i, N, OH, OW, OC);
        }
        const long long K = (long long)KH * KW * IC;
        const int8_t* w = b.const_data<int8_t>(op.weights, (size_t)OC * K, "weights", i);
        if (!w) return b.status;
        if (op.in0_zp < -128 || op.in0_zp > 127) return b.fail(TB200_INVALID_ARGUMENT, "op %d: input_zp outside int8", i);
        std::vector<int32_t> wsum(OC, 0);
        std::vector<long long> acc_bound(OC, 0);  // |sum x * w| <= 128 * sum |w|
        for (int oc = 0; oc < OC; oc++) {
          int32_t s = 0;
          long long sabs = 0;
          for (long long k = 0; k < K; k++) {
            const int v = w[(size_t)oc * K + k];
            s += v;
            sabs += v < 0 ? -v : v;
          }
          wsum[oc] = s;
          acc_bound[oc] = 128 * sabs;
        }
        std::vector<ChanParams> cp;
        int dr = 0;
        if (!b.chan_params(op, i, OC, wsum.data(), K, true, cp, dr)) return b.status;

        // 1x1 / fully_connected with symmetric weights: row-major GEMM on the tensor cores
        const bool pointwise = fc || (KH == 1 && KW == 1 && op.stride_h == 1 && op.stride_w == 1 && op.pad_t == 0 &&
                                      op.pad_b == 0 && op.pad_l == 0 && op.pad_r == 0);
        const long long M = (long long)N * OH * OW;
        // At most four rows: a weight-streaming dp4a kernel instead of 128-row tensor-core tiles (the weights are the
        // only traffic that counts there; 4 x K bytes of activations fit any SM's shared memory up to K = 12288)
        if (pointwise && op.weight_zp == 0 && !force_simt() && M <= 4 && K % 16 == 0 && K <= 12288) {
          FcRowsArgs fa{};
          fa.M = (int)M; fa.N = OC; fa.K = (int)K;
          fa.out_zp = op.out_zp; fa.clamp_min = op.clamp_min; fa.clamp_max = op.clamp_max; fa.hi_shift = b.last_hi_shift;
          const size_t w_off = b.add_const(w, (size_t)OC * K);
          const size_t c_off = b.add_const(cp.data(), cp.size() * sizeof(ChanParams));
          Loc lx = loc(op.in0), lo = loc(result_id);
          step.kernel_name = "fc_rows_dp4a";
          step.launch = [=](const ExecContext& c) {
            FcRowsArgs k = fa;
            k.x = (const int8_t*)lx.resolve(c);
            k.out = (int8_t*)lo.resolve(c);
            k.w = (const int8_t*)(c.consts + w_off);
            k.chan = (const ChanParams*)(c.consts + c_off);
            k.lut = has_lut ? (const int8_t*)(c.consts + lut_off) : nullptr;
            launch_fc_rows(k, c.stream);
          };
          break;
        }
        const int rgroup = pointwise_row_group(M, K, OC);
        if (pointwise && op.weight_zp == 0 && !force_simt() && rgroup <= 8 && M % rgroup == 0 &&
            (long long)OC * rgroup <= 65536 && gemm_tc_supported(M / rgroup, OC * rgroup, (int)K * rgroup, K * rgroup)) {
          GemmTcArgs ga{};
          const int Ng = OC * rgroup, Kg = (int)K * rgroup;
          const GemmTcGeometry geo = gemm_tc_geometry(Ng, Kg, M / rgroup);
          ga.M = M / rgroup; ga.N = Ng; ga.K = Kg;
          ga.lda = Kg; ga.ldc = Ng;
          ga.out_zp = op.out_zp; ga.clamp_min = op.clamp_min; ga.clamp_max = op.clamp_max;
          std::vector<int4> q4;
          ga.epi = Builder::q4_params(cp, acc_bound, dr != 0, op.out_zp, op.clamp_min, q4);
          const int rows = geo.n_tiles * geo.BN;
          std::vector<int8_t> wp((size_t)rows * geo.Kpad, 0);
          for (int j = 0; j < rgroup; j++)
            for (int oc = 0; oc < OC; oc++)
              memcpy(wp.data() + (size_t)(j * OC + oc) * geo.Kpad + (size_t)j * K, w + (size_t)oc * K, (size_t)K);
          {
            std::vector<ChanParams> rep((size_t)Ng);
            for (int j = 0; j < rgroup; j++)
              for (int oc = 0; oc < OC; oc++) rep[(size_t)j * OC + oc] = cp[oc];
            cp.swap(rep);
          }
          { ChanParams z{}; z.shift = 34; z.hshift = 2; z.rnd = 1ll << 33; cp.resize(rows, z); }
          size_t w_off = b.add_const(wp.data(), wp.size());
          size_t c_off = b.add_const(cp.data(), cp.size() * sizeof(ChanParams));
          size_t q_off = 0;
          if (ga.epi) {
            std::vector<int4> rep((size_t)rows, make_int4(0, 0, 0, 1));
            for (int j = 0; j < rgroup; j++)
              for (int oc = 0; oc < OC; oc++) rep[(size_t)j * OC + oc] = q4[oc];
            q_off = b.add_const(rep.data(), rep.size() * sizeof(int4));
          }
          const bool has_q4 = ga.epi != 0;
          // a residual add fused behind the product: the result is the add's, the other operand is read in the epilogue
          const int fused_add = add_after[i];
          int out_id = result_id;
          Loc lres{};
          if (fused_add >= 0) {
            if (!binary_args_of(ops[fused_add], ga.add) || ga.add.epi == 0)
              return b.fail(TB200_INTERNAL, "op %d: fused add lost its 32-bit rescale", fused_add);
            ga.add_self_is_a = add_self_is_a[i];
            out_id = ops[fused_add].out0;
            lres = loc(add_self_is_a[i] ? ops[fused_add].in1 : ops[fused_add].in0);
          }
          Loc lx = loc(op.in0), lo = loc(out_id);
          std::shared_ptr<GemmTcState> st(gemm_tc_state_new(), gemm_tc_state_free);
          step.kernel_name = "gemm_i8_tcgen05";
          step.launch = [=](const ExecContext& c) {
            GemmTcArgs k = ga;
            k.a = (const int8_t*)lx.resolve(c);
            k.out = (int8_t*)lo.resolve(c);
            k.w = (const int8_t*)(c.consts + w_off);
            k.chan = (const ChanParams*)(c.consts + c_off);
            k.q4 = has_q4 ? (const int4*)(c.consts + q_off) : nullptr;
            k.status = c.status;
            k.lut = has_lut ? (const int8_t*)(c.consts + lut_off) : nullptr;
            k.res = fused_add >= 0 ? (const int8_t*)lres.resolve(c) : nullptr;
            launch_gemm_i8_tc(k, st.get(), c.stream);
          };
          break;
        }

        if (add_after[i] >= 0) return b.fail(TB200_INTERNAL, "op %d: an add was fused into a convolution that does not take the GEMM", i);
        // Pixel groups for narrow stride-1 3-wide kernels (16 or 32 input channels, width a multiple of the group, one
        // pixel of padding left and right): the copy engine works row by row, a row being one pixel's channels, so 16-
        // and 32-byte pixels cost as much per row as 128-byte ones. The same convolution on the tensors read as
        // [N, H, W / G, G C] -> [N, OH, OW / G, G OC] (identical memory) is again a KH x 3 convolution with one group
        // of padding, its weights the original ones placed at [(j, oc)][kh][kp][(h, c)] and zero elsewhere. 1 / G of
        // the rows per pixel through the copy engine; the zero parts cost tensor-core work that is free here. Border classes, bias folding and the
        // epilogue constants follow from the transformed op as for any convolution.
        std::vector<int8_t> w_pairs;
        static const bool no_pairs = getenv("TB200_CONV_NO_PAIRS") != nullptr;  // A/B switch
        int group = 0;  // pixels per row of the rewritten convolution: 4 for 16 channels where the width allows, else 2
        if (!fc && !pointwise && !no_pairs && op.weight_zp == 0 && !force_simt() && op.stride_h == 1 && op.stride_w == 1 &&
            op.dil_h == 1 && op.dil_w == 1 && KW == 3 && KH <= 5 && op.pad_l == 1 && op.pad_r == 1 && (IC == 16 || IC == 32) &&
            OC % 16 == 0) {
          for (int g : {4, 2}) {
            if (W % g != 0 || IC * g > 64 || OC * g > 256) continue;
            if (conv_tc_supported(N, H, W / g, g * IC, g * OC, KH, 3, 1, 1, 1, 1, OH, OW / g) &&
                conv_tc_geometry_padded(N, OH, OW / g, W / g, g * IC, g * OC, KH, 3, 1, 1).halo) {
              group = g;
              break;
            }
          }
        }
        if (group) {
          const int G = group;
          // output pixel G P + j reads input pixel G (P + kp - 1) + h for kw = G (kp - 1) + h - j + 1
          w_pairs.assign((size_t)G * OC * KH * 3 * G * IC, 0);
          for (int j = 0; j < G; j++)
            for (int oc = 0; oc < OC; oc++)
              for (int kh = 0; kh < KH; kh++)
                for (int kp = 0; kp < 3; kp++)
                  for (int h = 0; h < G; h++) {
                    const int kw = G * (kp - 1) + h - j + 1;
                    if (kw < 0 || kw >= 3) continue;
                    memcpy(w_pairs.data() + ((((size_t)(j * OC + oc) * KH + kh) * 3 + kp) * G + h) * IC,
                           w + (((size_t)oc * KH + kh) * 3 + kw) * IC, (size_t)IC);
                  }
          {
            std::vector<ChanParams> cp2((size_t)G * OC);
            std::vector<long long> ab2((size_t)G * OC);
            for (int j = 0; j < G; j++)
              for (int oc = 0; oc < OC; oc++) {
                cp2[(size_t)j * OC + oc] = cp[oc];
                ab2[(size_t)j * OC + oc] = acc_bound[oc];
              }
            cp.swap(cp2);
            acc_bound.swap(ab2);
          }
          w = w_pairs.data();
          IC *= G; OC *= G; W /= G; OW /= G;
        }
        // KH x KW convolution with symmetric weights: implicit GEMM on the tensor cores (one TMA box per
        // tap and channel block, taps accumulated in TMEM; see gemm_tcgen05.cu)
        // (16 input channels with a load per tap or per kernel column: the copy engine's per-row cost makes 16-byte
        // rows a poor tensor-core operand and the direct dp4a kernel is faster; with one halo patch per tile the
        // row count no longer depends on the kernel size and the tensor cores take those too)
        if (!fc && !pointwise && op.weight_zp == 0 && !force_simt() &&
            conv_tc_supported(N, H, W, IC, OC, KH, KW, op.stride_h, op.stride_w, op.dil_h, op.dil_w, OH, OW) &&
            (IC != 16 || conv_tc_geometry_padded(N, OH, OW, W, IC, OC, KH, KW, op.stride_h, op.pad_l).halo ||
             conv_tc_geometry_padded(N, OH, OW, W, IC, OC, KH, KW, op.stride_h, op.pad_l).s2)) {
          const ConvTcGeometry geo = conv_tc_geometry_padded(N, OH, OW, W, IC, OC, KH, KW, op.stride_h, op.pad_l);
          ConvTcArgs ca{};
          ca.N = N; ca.H = H; ca.W = W; ca.IC = IC; ca.OC = OC; ca.KH = KH; ca.KW = KW; ca.OH = OH; ca.OW = OW;
          ca.stride = op.stride_h; ca.pad_t = op.pad_t; ca.pad_l = op.pad_l;
          ca.out_zp = op.out_zp; ca.clamp_min = op.clamp_min; ca.clamp_max = op.clamp_max;
          std::vector<int4> q4;
          {
            // the kernel adds a border correction of at most |izp| * sum |w| to the accumulator
            std::vector<long long> bound(acc_bound);
            for (auto& v : bound) v *= 2;
            ca.epi = Builder::q4_params(cp, bound, dr != 0, op.out_zp, op.clamp_min, q4);
          }
          const int rows = geo.n_tiles * geo.BN;
          std::vector<int8_t> wp((size_t)rows * geo.Kpad, 0);
          // OHWI rows are already in (kh, kw, ic) order; every tap is padded to whole channel blocks
          {
            const size_t tap_pad = (size_t)geo.icb_per_tap * geo.row_bytes;
            for (int oc = 0; oc < OC; oc++)
              for (int t = 0; t < KH * KW; t++)
                memcpy(wp.data() + (size_t)oc * geo.Kpad + t * tap_pad, w + ((size_t)oc * KH * KW + t) * IC, (size_t)IC);
          }
          { ChanParams z{}; z.shift = 34; z.hshift = 2; z.rnd = 1ll << 33; cp.resize(rows, z); }
          // Border classes. The copy engine fills taps outside the frame with 0 where the op means the
          // input zero point; cp's bias assumed izp for every tap, so a pixel gets back
          // izp * (weights of its outside taps).
          std::vector<uint8_t> rcls(OH), ccls(OW), nonzero;
          std::vector<uint32_t> rmasks, cmasks;
          auto classify = [](int out_dim, int in_dim, int k, int stride, int pad, std::vector<uint8_t>& cls,
                             std::vector<uint32_t>& masks) {
            for (int o = 0; o < out_dim; o++) {
              uint32_t m = 0;
              for (int t = 0; t < k; t++) {
                const int i = o * stride + t - pad;
                if (i < 0 || i >= in_dim) m |= 1u << t;
              }
              size_t id = 0;
              while (id < masks.size() && masks[id] != m) id++;
              if (id == masks.size()) masks.push_back(m);
              cls[o] = (uint8_t)id;
            }
          };
          classify(OH, H, KH, op.stride_h, op.pad_t, rcls, rmasks);
          classify(OW, W, KW, op.stride_w, op.pad_l, ccls, cmasks);
          std::vector<int32_t> corr;
          const bool need_corr = op.in0_zp != 0 && (rmasks.size() > 1 || cmasks.size() > 1 || rmasks[0] || cmasks[0]);
          if (need_corr) {
            if (rmasks.size() * cmasks.size() > 255) return b.fail(TB200_UNIMPLEMENTED, "op %d: too many border classes", i);
            corr.assign(rmasks.size() * cmasks.size() * (size_t)rows, 0);
            nonzero.assign(rmasks.size() * cmasks.size(), 0);
            for (size_t rc = 0; rc < rmasks.size(); rc++)
              for (size_t cc = 0; cc < cmasks.size(); cc++) {
                const size_t cls = rc * cmasks.size() + cc;
                for (int oc = 0; oc < OC; oc++) {
                  int32_t sum = 0;
                  for (int kh = 0; kh < KH; kh++)
                    for (int kw = 0; kw < KW; kw++)
                      if ((rmasks[rc] >> kh & 1) || (cmasks[cc] >> kw & 1)) {
                        const int8_t* tap = w + ((size_t)oc * KH * KW + (size_t)kh * KW + kw) * IC;
                        for (int ic = 0; ic < IC; ic++) sum += tap[ic];
                      }
                  const int32_t v = (int32_t)((uint32_t)op.in0_zp * (uint32_t)sum);
                  corr[cls * rows + oc] = v;
                  if (v) nonzero[cls] = 1;
                }
              }
          }
          const size_t w_off = b.add_const(wp.data(), wp.size());
          const size_t c_off = b.add_const(cp.data(), cp.size() * sizeof(ChanParams));
          size_t q_off = 0;
          if (ca.epi) {
            q4.resize(rows, make_int4(0, 0, 0, 1));
            q_off = b.add_const(q4.data(), q4.size() * sizeof(int4));
          }
          const bool has_q4 = ca.epi != 0;
          size_t corr_off = 0, rcls_off = 0, ccls_off = 0, nz_off = 0;
          if (need_corr) {
            corr_off = b.add_const(corr.data(), corr.size() * 4);
            rcls_off = b.add_const(rcls.data(), rcls.size());
            ccls_off = b.add_const(ccls.data(), ccls.size());
            nz_off = b.add_const(nonzero.data(), nonzero.size());
            ca.ncc = (int)cmasks.size();
          }
          Loc lx = loc(op.in0), lo = loc(result_id);
          std::shared_ptr<GemmTcState> st(gemm_tc_state_new(), gemm_tc_state_free);
          step.kernel_name = "conv_igemm_i8_tcgen05";
          step.launch = [=](const ExecContext& c) {
            ConvTcArgs k = ca;
            k.x = (const int8_t*)lx.resolve(c);
            k.out = (int8_t*)lo.resolve(c);
            k.w = (const int8_t*)(c.consts + w_off);
            k.chan = (const ChanParams*)(c.consts + c_off);
            k.q4 = has_q4 ? (const int4*)(c.consts + q_off) : nullptr;
            if (need_corr) {
              k.corr = (const int32_t*)(c.consts + corr_off);
              k.rcls = (const uint8_t*)(c.consts + rcls_off);
              k.ccls = (const uint8_t*)(c.consts + ccls_off);
              k.cls_nonzero = (const uint8_t*)(c.consts + nz_off);
            }
            k.status = c.status;
            k.lut = has_lut ? (const int8_t*)(c.consts + lut_off) : nullptr;
            const cudaError_t e = launch_conv_i8_tc(k, st.get(), c.stream);
            if (e != cudaSuccess && c.launch_error) *c.launch_error = e;
          };
          break;
        }

        const int Kpad = (int)((K + 31) / 32 * 32);
        std::vector<int8_t> packed((size_t)OC * Kpad, 0);
        for (int oc = 0; oc < OC; oc++) memcpy(packed.data() + (size_t)oc * Kpad, w + (size_t)oc * K, (size_t)K);
        ConvArgs a{};
        a.N = N; a.H = H; a.W = W; a.IC = IC; a.OC = OC; a.KH = KH; a.KW = KW; a.OH = OH; a.OW = OW;
        a.stride_h = fc ? 1 : op.stride_h; a.stride_w = fc ? 1 : op.stride_w;
        a.dil_h = fc ? 1 : op.dil_h; a.dil_w = fc ? 1 : op.dil_w;
        a.pad_t = fc ? 0 : op.pad_t; a.pad_l = fc ? 0 : op.pad_l;
        a.K = (int)K; a.Kpad = Kpad;
        a.input_zp = op.in0_zp; a.weight_zp = op.weight_zp; a.out_zp = op.out_zp;
        a.clamp_min = op.clamp_min; a.clamp_max = op.clamp_max; a.double_round = dr; a.hi_shift = b.last_hi_shift;
        size_t w_off = b.add_const(packed.data(), packed.size());
        size_t c_off = b.add_const(cp.data(), cp.size() * sizeof(ChanParams));
        // the compact 32-bit records, for the CUDA-core kernels that take them (the 3x3x3 stem)
        std::vector<int4> q4s;
        a.epi = fc ? 0 : Builder::q4_params(cp, acc_bound, dr != 0, op.out_zp, op.clamp_min, q4s);
        const size_t q_off = a.epi ? b.add_const(q4s.data(), q4s.size() * sizeof(int4)) : 0;
        const bool has_q4s = a.epi != 0;
        a.x_bytes = (long long)b.numel(op.in0);
        Loc lx = loc(op.in0), lo = loc(result_id);
        step.kernel_name = conv2d_simt_kernel_name(a);
        step.launch = [=](const ExecContext& c) {
          ConvArgs k = a;
          k.x = (const int8_t*)lx.resolve(c);
          k.out = (int8_t*)lo.resolve(c);
          k.w = (const int8_t*)(c.consts + w_off);
          k.chan = (const ChanParams*)(c.consts + c_off);
          k.q4 = has_q4s ? (const int4*)(c.consts + q_off) : nullptr;
          k.lut = has_lut ? (const int8_t*)(c.consts + lut_off) : nullptr;
          launch_conv2d_simt(k, c.stream);
        };
        break;
      }
      case TB200_OP_DEPTHWISE: {
        if (!b.act_i8(op.in0, 4) || !b.act_i8(op.out0, 4) || !b.valid_id(op.weights) || tensors[op.weights].rank != 4)
          return b.fail(TB200_INVALID_ARGUMENT, "op %d: depthwise wants int8 NHWC input/output and [KH,KW,C,M] weights", i);
        const auto& x = tensors[op.in0]; const auto& w = tensors[op.weights]; const auto& o = tensors[op.out0];
        DwArgs a{};
        a.N = x.shape[0]; a.H = x.shape[1]; a.W = x.shape[2]; a.C = x.shape[3];
        a.KH = w.shape[0]; a.KW = w.shape[1]; a.M = w.shape[3];
        if (w.shape[2] != a.C) return b.fail(TB200_INVALID_ARGUMENT, "op %d: depthwise weight C mismatch", i);
        if (op.stride_h < 1 || op.stride_w < 1 || op.dil_h < 1 || op.dil_w < 1 || op.pad_t < 0 || op.pad_b < 0 ||
            op.pad_l < 0 || op.pad_r < 0)
          return b.fail(TB200_INVALID_ARGUMENT, "op %d: bad stride/dilation/pad", i);
        a.OH = conv_out_dim(a.H, a.KH, op.stride_h, op.dil_h, op.pad_t, op.pad_b);
        a.OW = conv_out_dim(a.W, a.KW, op.stride_w, op.dil_w, op.pad_l, op.pad_r);
        const int OC = a.C * a.M;
        if (o.shape[0] != a.N || o.shape[1] != a.OH || o.shape[2] != a.OW || o.shape[3] != OC)
          return b.fail(TB200_INVALID_ARGUMENT, "op %d: depthwise output shape mismatch", i);
        const int8_t* wd = b.const_data<int8_t>(op.weights, (size_t)a.KH * a.KW * OC, "weights", i);
        if (!wd) return b.status;
        a.stride_h = op.stride_h; a.stride_w = op.stride_w; a.dil_h = op.dil_h; a.dil_w = op.dil_w;
        a.pad_t = op.pad_t; a.pad_l = op.pad_l;
        a.input_zp = op.in0_zp; a.weight_zp = op.weight_zp; a.out_zp = op.out_zp;
        a.clamp_min = op.clamp_min; a.clamp_max = op.clamp_max;
        if (op.in0_zp < -128 || op.in0_zp > 127) return b.fail(TB200_INVALID_ARGUMENT, "op %d: input_zp outside int8", i);
        // the 3x3 dp4a kernel stages izp for taps outside the image and wants -izp * sum(w) in the bias
        const bool fast = depthwise3x3_supported(a) && !force_simt();
        std::vector<int32_t> wsum;
        if (fast) {
          wsum.assign(OC, 0);
          for (int t = 0; t < 9; t++)
            for (int ch = 0; ch < OC; ch++) wsum[ch] += wd[(size_t)t * OC + ch];
        }
        std::vector<ChanParams> cp;
        int dr = 0;
        if (!b.chan_params(op, i, OC, fast ? wsum.data() : nullptr, 9, fast, cp, dr)) return b.status;
        a.double_round = dr; a.hi_shift = b.last_hi_shift;
        std::vector<int4> q4;
        if (fast) {
          // nine taps: |acc| <= 128 * sum |w| (taps outside the image are staged as the zero point and add nothing)
          std::vector<long long> bound(OC, 0);
          for (int t = 0; t < 9; t++)
            for (int ch = 0; ch < OC; ch++) bound[ch] += 128 * (long long)std::abs((int)wd[(size_t)t * OC + ch]);
          a.epi = Builder::q4_params(cp, bound, dr != 0, op.out_zp, op.clamp_min, q4);
        }
        size_t w_off = b.add_const(wd, (size_t)a.KH * a.KW * OC);
        size_t c_off = b.add_const(cp.data(), cp.size() * sizeof(ChanParams));
        size_t q_off = 0, q4_off = 0;
        if (fast) {
          std::vector<uint32_t> wq((size_t)3 * 2 * OC);
          size_t nw = depthwise3x3_pack(wd, OC, op.stride_h, wq.data());
          q_off = b.add_const(wq.data(), nw * sizeof(uint32_t));
          if (a.epi) q4_off = b.add_const(q4.data(), q4.size() * sizeof(int4));
        }
        const bool has_q4 = a.epi != 0;
        Loc lx = loc(op.in0), lo = loc(op.out0);
        step.kernel_name = fast ? "depthwise3x3_dp4a" : "depthwise";
        step.launch = [=](const ExecContext& c) {
          DwArgs k = a;
          k.x = (const int8_t*)lx.resolve(c);
          k.out = (int8_t*)lo.resolve(c);
          k.w = (const int8_t*)(c.consts + w_off);
          k.chan = (const ChanParams*)(c.consts + c_off);
          k.wq = fast ? (const uint32_t*)(c.consts + q_off) : nullptr;
          k.q4 = has_q4 ? (const int4*)(c.consts + q4_off) : nullptr;
          launch_depthwise(k, c.stream);
        };
        break;
      }
      case TB200_OP_MATMUL_I32: {
        if (op.weights < 0 && op.in1 >= 0) {
          // both operands are runtime tensors (the form of the reference's tosa.matmul fixtures): int8 x int8 or
          // int16 x int16, int32 or int16 result
          if (!b.valid_id(op.in0) || !b.valid_id(op.in1) || !b.valid_id(op.out0))
            return b.fail(TB200_INVALID_ARGUMENT, "op %d: bad tensor id", i);
          const auto& ta = tensors[op.in0]; const auto& tb = tensors[op.in1]; const auto& to = tensors[op.out0];
          const bool in16 = ta.dtype == TB200_I16, out16 = to.dtype == TB200_I16;
          if ((ta.dtype != TB200_I8 && !in16) || tb.dtype != ta.dtype || (to.dtype != TB200_I32 && !out16) || ta.rank != 2 ||
              tb.rank != 2 || to.rank != 2)
            return b.fail(TB200_INVALID_ARGUMENT, "op %d: matmul wants [M,K] x [K,N] of int8 or int16 -> int32 or int16 [M,N]", i);
          const int M = ta.shape[0], K = ta.shape[1], N = tb.shape[1];
          if (tb.shape[0] != K || to.shape[0] != M || to.shape[1] != N)
            return b.fail(TB200_INVALID_ARGUMENT, "op %d: matmul shape mismatch", i);
          Loc lx = loc(op.in0), lw = loc(op.in1), lo = loc(op.out0);
          const int azp = op.in0_zp, bzp = op.weight_zp;
          step.kernel_name = "matmul_int";
          step.launch = [=](const ExecContext& c) {
            launch_matmul_int(lx.resolve(c), lw.resolve(c), lo.resolve(c), in16, out16, M, K, N, azp, bzp, c.stream);
          };
          break;
        }
        if (!b.act_i8(op.in0, 2) || !b.valid_id(op.weights) || tensors[op.weights].rank != 2 || !b.valid_id(op.out0) ||
            tensors[op.out0].dtype != TB200_I32 || tensors[op.out0].rank != 2)
          return b.fail(TB200_INVALID_ARGUMENT, "op %d: matmul wants int8 [M,K] x const int8 [K,N] -> int32 [M,N]", i);
        int M = tensors[op.in0].shape[0], K = tensors[op.in0].shape[1], N = tensors[op.weights].shape[1];
        if (tensors[op.weights].shape[0] != K || tensors[op.out0].shape[0] != M || tensors[op.out0].shape[1] != N)
          return b.fail(TB200_INVALID_ARGUMENT, "op %d: matmul shape mismatch", i);
        const int8_t* wd = b.const_data<int8_t>(op.weights, (size_t)K * N, "weights", i);
        if (!wd) return b.status;
        size_t w_off = b.add_const(wd, (size_t)K * N);
        Loc lx = loc(op.in0), lo = loc(op.out0);
        int azp = op.in0_zp, bzp = op.weight_zp;
        step.kernel_name = "matmul_int";
        step.launch = [=](const ExecContext& c) {
          launch_matmul_int(lx.resolve(c), c.consts + w_off, lo.resolve(c), false, false, M, K, N, azp, bzp, c.stream);
        };
        break;
      }
      case TB200_OP_MAXPOOL:
      case TB200_OP_AVGPOOL: {
        // max pool also takes int16 tensors (the reference's MaxPool2D i16 -> i16)
        const bool pool16 = op.kind == TB200_OP_MAXPOOL && b.valid_id(op.in0) && b.valid_id(op.out0) &&
                            tensors[op.in0].dtype == TB200_I16 && tensors[op.out0].dtype == TB200_I16 &&
                            tensors[op.in0].rank == 4 && tensors[op.out0].rank == 4 &&
                            tensors[op.in0].kind != TB200_TENSOR_CONSTANT;
        if (!pool16 && (!b.act_i8(op.in0, 4) || !b.act_i8(op.out0, 4)))
          return b.fail(TB200_INVALID_ARGUMENT, "op %d: pooling wants int8 NHWC input/output (max pool: or int16)", i);
        const auto& x = tensors[op.in0]; const auto& o = tensors[op.out0];
        PoolArgs a{};
        a.elem16 = pool16 ? 1 : 0;
        a.N = x.shape[0]; a.H = x.shape[1]; a.W = x.shape[2]; a.C = x.shape[3];
        a.KH = op.kh; a.KW = op.kw; a.stride_h = op.stride_h; a.stride_w = op.stride_w;
        a.pad_t = op.pad_t; a.pad_l = op.pad_l;
        if (a.KH < 1 || a.KW < 1 || a.stride_h < 1 || a.stride_w < 1 || op.pad_t < 0 || op.pad_b < 0 || op.pad_l < 0 ||
            op.pad_r < 0)
          return b.fail(TB200_INVALID_ARGUMENT, "op %d: bad pooling window", i);
        a.OH = conv_out_dim(a.H, a.KH, a.stride_h, 1, op.pad_t, op.pad_b);
        a.OW = conv_out_dim(a.W, a.KW, a.stride_w, 1, op.pad_l, op.pad_r);
        if (o.shape[0] != a.N || o.shape[1] != a.OH || o.shape[2] != a.OW || o.shape[3] != a.C)
          return b.fail(TB200_INVALID_ARGUMENT, "op %d: pooling output shape mismatch", i);
        a.pad_value = op.pad_value; a.input_zp = op.in0_zp; a.output_zp = op.out_zp;
        Loc lx = loc(op.in0), lo = loc(op.out0);
        const bool is_max = op.kind == TB200_OP_MAXPOOL;
        if (!is_max && (long long)a.KH * a.KW > 256)  // the kernel's per-count rescale table
          return b.fail(TB200_UNIMPLEMENTED, "op %d: average pooling windows above 256 taps are not supported", i);
        step.kernel_name = is_max ? "maxpool" : "avgpool";
        step.launch = [=](const ExecContext& c) {
          PoolArgs k = a;
          k.x = (const int8_t*)lx.resolve(c);
          k.out = (int8_t*)lo.resolve(c);
          if (is_max) launch_maxpool(k, c.stream);
          else launch_avgpool(k, c.stream);
        };
        break;
      }
      case TB200_OP_ADD:
      case TB200_OP_SUB:
      case TB200_OP_MUL: {
        if (!b.valid_id(op.in0) || !b.valid_id(op.in1) || !b.valid_id(op.out0) || tensors[op.in0].dtype != TB200_I8 ||
            tensors[op.in1].dtype != TB200_I8 || tensors[op.out0].dtype != TB200_I8)
          return b.fail(TB200_INVALID_ARGUMENT, "op %d: elementwise op wants int8 operands", i);
        size_t n = b.numel(op.in0);
        if (b.numel(op.in1) != n || b.numel(op.out0) != n)
          return b.fail(TB200_INVALID_ARGUMENT, "op %d: elementwise operands differ in size (no broadcast)", i);
        for (int s : {op.in0_shift, op.in1_shift, op.out_shift})
          if (s < 2 || s > 62) return b.fail(TB200_INVALID_ARGUMENT, "op %d: rescale shift %d outside [2,62]", i, s);
        BinaryArgs a{};
        if (!binary_args_of(op, a)) return b.fail(TB200_INVALID_ARGUMENT, "op %d: input left shift outside [0,22]", i);
        a.n = (long long)n;
        Loc la = loc(op.in0), lb = loc(op.in1), lo = loc(op.out0);
        step.kernel_name = "binary_rescale";
        step.launch = [=](const ExecContext& c) {
          BinaryArgs k = a;
          k.a = (const int8_t*)la.resolve(c);
          k.b = (const int8_t*)lb.resolve(c);
          k.out = (int8_t*)lo.resolve(c);
          launch_binary(k, c.stream);
        };
        break;
      }
      case TB200_OP_TABLE: {
        if (!b.valid_id(op.in0) || !b.valid_id(op.out0) || tensors[op.in0].dtype != TB200_I8 ||
            tensors[op.out0].dtype != TB200_I8 || b.numel(op.in0) != b.numel(op.out0))
          return b.fail(TB200_INVALID_ARGUMENT, "op %d: table wants int8 input/output of equal size", i);
        const int8_t* tbl = b.const_data<int8_t>(op.table, 256, "table", i);
        if (!tbl) return b.status;
        size_t t_off = b.add_const(tbl, 256);
        long long n = (long long)b.numel(op.in0);
        Loc lx = loc(op.in0), lo = loc(op.out0);
        step.kernel_name = "table";
        step.launch = [=](const ExecContext& c) {
          launch_table((const int8_t*)lx.resolve(c), (const int8_t*)(c.consts + t_off), (int8_t*)lo.resolve(c), n,
                       c.stream);
        };
        break;
      }
      case TB200_OP_RESCALE: {
        if (!b.valid_id(op.in0) || !b.valid_id(op.out0) || b.numel(op.in0) != b.numel(op.out0))
          return b.fail(TB200_INVALID_ARGUMENT, "op %d: rescale wants input/output of equal size", i);
        if (tensors[op.in0].dtype != TB200_I8 || tensors[op.out0].dtype != TB200_I8 || op.flags != 0) {
          // generic form: any of i8 / i16 / i32 in and out, unsigned storage by flag
          auto int_t = [](uint32_t d) { return d == TB200_I8 || d == TB200_I16 || d == TB200_I32; };
          if (!int_t(tensors[op.in0].dtype) || !int_t(tensors[op.out0].dtype))
            return b.fail(TB200_INVALID_ARGUMENT, "op %d: rescale wants integer tensors", i);
          const auto& x = tensors[op.in0];
          const int C = x.shape[x.rank - 1];
          const int nscale = op.per_channel ? C : 1;
          const int32_t* mult = b.const_data<int32_t>(op.multiplier, nscale, "multiplier", i);
          const int8_t* shift = b.const_data<int8_t>(op.shift, nscale, "shift", i);
          if (!mult || !shift) return b.status;
          for (int c = 0; c < nscale; c++)
            if (shift[c] < 2 || shift[c] > 62) return b.fail(TB200_INVALID_ARGUMENT, "op %d: rescale shift %d outside [2,62]", i, (int)shift[c]);
          RescaleGenericArgs a{};
          a.n = (long long)b.numel(op.in0); a.C = C; a.per_channel = op.per_channel;
          a.in_dtype = x.dtype; a.out_dtype = tensors[op.out0].dtype;
          a.input_unsigned = (op.flags & TB200_FLAG_INPUT_UNSIGNED) ? 1 : 0;
          a.in_zp = op.in0_zp; a.out_zp = op.out_zp; a.double_round = op.double_round;
          a.clamp_min = op.clamp_min; a.clamp_max = op.clamp_max;
          if (op.flags & TB200_FLAG_OUTPUT_UNSIGNED) a.clamp_max = (long long)(uint32_t)op.clamp_max;
          const size_t m_off = b.add_const(mult, (size_t)nscale * 4), s_off = b.add_const(shift, (size_t)nscale);
          Loc lx = loc(op.in0), lo = loc(op.out0);
          step.kernel_name = "rescale_generic";
          step.launch = [=](const ExecContext& c) {
            RescaleGenericArgs k = a;
            k.x = lx.resolve(c); k.out = lo.resolve(c);
            k.mult = (const int32_t*)(c.consts + m_off); k.shift = (const int8_t*)(c.consts + s_off);
            launch_rescale_generic(k, c.stream);
          };
          break;
        }
        const auto& x = tensors[op.in0];
        int C = x.shape[x.rank - 1];
        std::vector<ChanParams> cp;
        int dr = 0;
        if (!b.chan_params(op, i, op.per_channel ? C : 1, nullptr, 0, false, cp, dr)) return b.status;
        RescaleArgs a{};
        a.rows = (long long)(b.numel(op.in0) / C); a.C = C; a.per_channel = op.per_channel;
        a.input_zp = op.in0_zp; a.out_zp = op.out_zp; a.clamp_min = op.clamp_min; a.clamp_max = op.clamp_max;
        a.double_round = dr; a.out_row_stride = C; a.out_col_offset = 0;
        size_t c_off = b.add_const(cp.data(), cp.size() * sizeof(ChanParams));
        Loc lx = loc(op.in0), lo = loc(op.out0);
        step.kernel_name = "rescale";
        step.launch = [=](const ExecContext& c) {
          RescaleArgs k = a;
          k.x = (const int8_t*)lx.resolve(c);
          k.out = (int8_t*)lo.resolve(c);
          k.chan = (const ChanParams*)(c.consts + c_off);
          launch_rescale(k, c.stream);
        };
        break;
      }
      case TB200_OP_CONCAT: {
        if (!b.valid_id(op.in0) || !b.valid_id(op.in1) || !b.valid_id(op.out0) || tensors[op.in0].dtype != TB200_I8 ||
            tensors[op.in1].dtype != TB200_I8 || tensors[op.out0].dtype != TB200_I8)
          return b.fail(TB200_INVALID_ARGUMENT, "op %d: concat wants int8 operands", i);
        const auto& x0 = tensors[op.in0]; const auto& x1 = tensors[op.in1]; const auto& o = tensors[op.out0];
        int C0 = x0.shape[x0.rank - 1], C1 = x1.shape[x1.rank - 1], CO = o.shape[o.rank - 1];
        size_t rows = b.numel(op.in0) / C0;
        if (C0 + C1 != CO || b.numel(op.in1) / C1 != rows || b.numel(op.out0) / CO != rows)
          return b.fail(TB200_INVALID_ARGUMENT, "op %d: concat (channel axis) shape mismatch", i);
        for (int s : {op.in0_shift, op.in1_shift})
          if (s < 2 || s > 62) return b.fail(TB200_INVALID_ARGUMENT, "op %d: rescale shift %d outside [2,62]", i, s);
        ChanParams p0{}, p1{};
        p0.mult = op.in0_mult; p0.shift = op.in0_shift; p1.mult = op.in1_mult; p1.shift = op.in1_shift;
        Builder::fill_rounding(p0, op.double_round != 0);
        Builder::fill_rounding(p1, op.double_round != 0);
        size_t c0_off = b.add_const(&p0, sizeof(p0));
        size_t c1_off = b.add_const(&p1, sizeof(p1));
        RescaleArgs a0{}, a1{};
        a0.rows = a1.rows = (long long)rows;
        a0.C = C0; a1.C = C1;
        a0.input_zp = op.in0_zp; a1.input_zp = op.in1_zp;
        a0.out_zp = a1.out_zp = op.out_zp;
        a0.clamp_min = a1.clamp_min = -128; a0.clamp_max = a1.clamp_max = 127;
        a0.double_round = a1.double_round = op.double_round;
        // chained concats are written in place (see concat_into): rows are as wide as the last result of
        // the chain, and an operand that is already in place is not copied
        int fin = op.out0;
        while (concat_into[fin] >= 0) fin = concat_into[fin];
        const int row_stride = tensors[fin].shape[tensors[fin].rank - 1];
        const bool in0_in_place = concat_into[op.in0] == op.out0;
        a0.out_row_stride = a1.out_row_stride = row_stride;
        a0.out_col_offset = 0; a1.out_col_offset = C0;
        a0.identity = op.in0_mult == (1 << 30) && op.in0_shift == 30 && op.in0_zp == op.out_zp;
        a1.identity = op.in1_mult == (1 << 30) && op.in1_shift == 30 && op.in1_zp == op.out_zp;
        Loc l0 = loc(op.in0), l1 = loc(op.in1), lo = loc(op.out0);
        step.kernel_name = "concat_rescale";
        step.launches = in0_in_place ? 1 : 2;
        step.launch = [=](const ExecContext& c) {
          RescaleArgs k0 = a0, k1 = a1;
          k0.x = (const int8_t*)l0.resolve(c); k1.x = (const int8_t*)l1.resolve(c);
          k0.out = k1.out = (int8_t*)lo.resolve(c);
          k0.chan = (const ChanParams*)(c.consts + c0_off);
          k1.chan = (const ChanParams*)(c.consts + c1_off);
          if (!in0_in_place) launch_rescale(k0, c.stream);
          launch_rescale(k1, c.stream);
        };
        break;
      }
      case TB200_OP_RESIZE_NN2X: {
        if (!b.act_i8(op.in0, 4) || !b.act_i8(op.out0, 4))
          return b.fail(TB200_INVALID_ARGUMENT, "op %d: resize wants int8 NHWC input/output", i);
        const auto& x = tensors[op.in0]; const auto& o = tensors[op.out0];
        int N = x.shape[0], H = x.shape[1], W = x.shape[2], C = x.shape[3];
        if (o.shape[0] != N || o.shape[1] != 2 * H || o.shape[2] != 2 * W || o.shape[3] != C)
          return b.fail(TB200_INVALID_ARGUMENT, "op %d: resize output must be 2x the input frame", i);
        Loc lx = loc(op.in0), lo = loc(op.out0);
        step.kernel_name = "resize_nn2x";
        step.launch = [=](const ExecContext& c) {
          launch_resize_nn2x((const int8_t*)lx.resolve(c), (int8_t*)lo.resolve(c), N, H, W, C, c.stream);
        };
        break;
      }
      case TB200_OP_EMBED: {
        if (!b.is_t(op.in0, TB200_I32, 1) || !b.is_t(op.out0, TB200_BF16, 2) || !b.valid_id(op.weights) ||
            tensors[op.weights].rank != 2)
          return b.fail(TB200_INVALID_ARGUMENT, "op %d: embed wants i32 [B] tokens, an int8 [V,H] table, bf16 [B,H] out", i);
        const int B = tensors[op.in0].shape[0], V = tensors[op.weights].shape[0], H = tensors[op.weights].shape[1];
        if (tensors[op.out0].shape[0] != B || tensors[op.out0].shape[1] != H)
          return b.fail(TB200_INVALID_ARGUMENT, "op %d: embed output shape mismatch", i);
        size_t w_off, s_off;
        if (!b.add_raw_const(op.weights, (size_t)V * H, "table", i, w_off)) return b.status;
        if (!b.add_raw_const(op.bias, (size_t)V * 2, "scales", i, s_off)) return b.status;
        Loc lt = loc(op.in0), lo = loc(op.out0);
        const float mult = op.f0;
        step.kernel_name = "embed_w8";
        step.launch = [=](const ExecContext& c) {
          launch_embed((const int32_t*)lt.resolve(c), (const int8_t*)(c.consts + w_off),
                       (const uint16_t*)(c.consts + s_off), (uint16_t*)lo.resolve(c), B, H, V, mult, c.stream);
        };
        break;
      }
      case TB200_OP_RMSNORM: {
        if (!b.is_t(op.in0, TB200_BF16, 2) || !b.is_t(op.out0, TB200_BF16, 2) || (op.in1 >= 0 && !b.is_t(op.in1, TB200_BF16, 2)))
          return b.fail(TB200_INVALID_ARGUMENT, "op %d: rmsnorm wants bf16 [rows,H] tensors", i);
        const int rows = tensors[op.in0].shape[0], H = tensors[op.in0].shape[1];
        if (b.numel(op.out0) != (size_t)rows * H || (op.in1 >= 0 && b.numel(op.in1) != (size_t)rows * H))
          return b.fail(TB200_INVALID_ARGUMENT, "op %d: rmsnorm shape mismatch", i);
        size_t w_off;
        if (!b.add_raw_const(op.weights, (size_t)H * 2, "norm weight", i, w_off)) return b.status;
        Loc lx = loc(op.in0), lr = loc(op.in1), lo = loc(op.out0);
        const float eps = op.f0;
        const bool has_res = op.in1 >= 0;
        const DeferredGemv dg = partials_of(i);
        const int second = norm_second[i];
        if (dg.splits > 0 || second >= 0) {
          size_t w2_off = 0;
          Loc lo2{};
          float eps2 = 0.f;
          if (second >= 0) {
            if (!b.add_raw_const(ops[second].weights, (size_t)H * 2, "norm weight", second, w2_off)) return b.status;
            lo2 = loc(ops[second].out0);
            eps2 = ops[second].f0;
          }
          step.kernel_name = second >= 0 ? (dg.splits > 0 ? "rmsnorm_pair_from_partials" : "rmsnorm_pair")
                                         : "rmsnorm_from_partials";
          step.launch = [=](const ExecContext& c) {
            const GemvPartials gp{dg.splits > 0 ? (const float*)c.scratch : nullptr,
                                  dg.splits > 0 ? (const uint16_t*)(c.consts + dg.scale_off) : nullptr, dg.splits};
            launch_rmsnorm_fused((const uint16_t*)lx.resolve(c), gp, has_res ? (const uint16_t*)lr.resolve(c) : nullptr,
                                 (const uint16_t*)(c.consts + w_off), (uint16_t*)lo.resolve(c),
                                 second >= 0 ? (const uint16_t*)(c.consts + w2_off) : nullptr,
                                 second >= 0 ? (uint16_t*)lo2.resolve(c) : nullptr, rows, H, eps, eps2, c.stream);
          };
          break;
        }
        step.kernel_name = "rmsnorm";
        step.launch = [=](const ExecContext& c) {
          launch_rmsnorm((const uint16_t*)lx.resolve(c), has_res ? (const uint16_t*)lr.resolve(c) : nullptr,
                         (const uint16_t*)(c.consts + w_off), (uint16_t*)lo.resolve(c), rows, H, eps, c.stream);
        };
        break;
      }
      case TB200_OP_GEMV_W8: {
        if (!b.is_t(op.in0, TB200_BF16, 2) || (!b.is_t(op.out0, TB200_BF16, 2) && !b.is_t(op.out0, TB200_F32, 2)) ||
            !b.valid_id(op.weights) || tensors[op.weights].rank != 2 || tensors[op.weights].dtype != TB200_I8)
          return b.fail(TB200_INVALID_ARGUMENT, "op %d: gemv_w8 wants bf16 [B,K] x int8 [N,K] -> bf16 or f32 [B,N]", i);
        const int y_f32 = tensors[op.out0].dtype == TB200_F32;
        const int B = tensors[op.in0].shape[0], N = tensors[op.weights].shape[0];
        // i1 > 0 or a narrower weight matrix: the product takes columns [i1, i1 + K) of the input (a tensor-
        // parallel shard whose K slice is part of a head); only the fused decode step implements that
        const int K = tensors[op.weights].shape[1];
        if (op.i1 < 0 || op.i1 + K > tensors[op.in0].shape[1] || tensors[op.out0].shape[0] != B || tensors[op.out0].shape[1] != N)
          return b.fail(TB200_INVALID_ARGUMENT, "op %d: gemv_w8 shape mismatch", i);
        if (op.i1 != 0 || K != tensors[op.in0].shape[1]) needs_fusion = true;
        if (K % 16 != 0 || B > 32) return b.fail(TB200_UNIMPLEMENTED, "op %d: gemv_w8 needs K %% 16 == 0 and batch <= 32", i);
        size_t w_off, s_off;
        if (!b.add_raw_const(op.weights, (size_t)N * K, "weights", i, w_off)) return b.status;
        if (!b.add_raw_const(op.bias, (size_t)N * 2, "scales", i, s_off)) return b.status;
        const int splits = op.i0 > 0 ? op.i0 : gemv_w8_splits(B, N, K);
        if (!gemv_w8_splits_fit(B, N, K, splits))
          return b.fail(TB200_OUT_OF_RANGE, "op %d: %d K slices leave a slice longer than the tensor-core gemv_w8 can stage", i, splits);
        scratch_need = std::max(scratch_need, gemv_w8_scratch_bytes(B, N, splits));
        Loc lx = loc(op.in0), lo = loc(op.out0);
        const bool finalize = !defer_finalize[i];
        if (!finalize) deferred[i] = DeferredGemv{s_off, gemv_w8_used_splits(B, N, K, splits)};
        step.kernel_name = !finalize ? "gemv_w8_splitk_partials" : splits > 1 ? "gemv_w8_splitk" : "gemv_w8";
        step.launches = splits > 1 && finalize ? 2 : 1;
        step.launch = [=](const ExecContext& c) {
          launch_gemv_w8((const uint16_t*)lx.resolve(c), (const int8_t*)(c.consts + w_off),
                         (const uint16_t*)(c.consts + s_off), lo.resolve(c), y_f32, (float*)c.scratch, B, N, K, splits,
                         c.stream, finalize);
        };
        break;
      }
      case TB200_OP_ROPE_KV: {
        const int n_q = op.i0, n_kv = op.i1, D = op.i2;
        if (!b.is_t(op.in0, TB200_BF16, 2) || !b.is_t(op.in1, TB200_I32, 1) || !b.is_t(op.out0, TB200_BF16, 2) ||
            !b.is_t(op.out1, TB200_BF16, 3) || !b.is_t(op.in2, TB200_BF16, 3) || n_q < 1 || n_kv < 1 || D < 2 || D > 512 ||
            (D & 1))
          return b.fail(TB200_INVALID_ARGUMENT, "op %d: rope_kv wants bf16 qkv [B,(q+2kv)*D], i32 pos, bf16 caches [B,T,kv*D]", i);
        const int B = tensors[op.in0].shape[0], T = tensors[op.out1].shape[1];
        if (tensors[op.in0].shape[1] != (n_q + 2 * n_kv) * D || tensors[op.out0].shape[0] != B ||
            tensors[op.out0].shape[1] != n_q * D || tensors[op.out1].shape[0] != B || tensors[op.out1].shape[2] != n_kv * D ||
            b.numel(op.in2) != b.numel(op.out1) || tensors[op.out1].kind != TB200_TENSOR_STATE ||
            tensors[op.in2].kind != TB200_TENSOR_STATE)
          return b.fail(TB200_INVALID_ARGUMENT, "op %d: rope_kv shape mismatch (caches must be state tensors)", i);
        size_t qw_off, kw_off;
        if (!b.add_raw_const(op.weights, (size_t)D * 2, "q_norm weight", i, qw_off)) return b.status;
        if (!b.add_raw_const(op.bias, (size_t)D * 2, "k_norm weight", i, kw_off)) return b.status;
        Loc lx = loc(op.in0), lp = loc(op.in1), lq = loc(op.out0), lk = loc(op.out1), lv = loc(op.in2);
        const float theta = op.f0, eps = op.f1;
        const DeferredGemv dg = partials_of(i);
        step.kernel_name = dg.splits > 0 ? "rope_kv_from_partials" : "rope_kv";
        step.launch = [=](const ExecContext& c) {
          const GemvPartials gp{dg.splits > 0 ? (const float*)c.scratch : nullptr,
                                dg.splits > 0 ? (const uint16_t*)(c.consts + dg.scale_off) : nullptr, dg.splits};
          launch_rope_kv((const uint16_t*)lx.resolve(c), (const int32_t*)lp.resolve(c), (const uint16_t*)(c.consts + qw_off),
                         (const uint16_t*)(c.consts + kw_off), (uint16_t*)lq.resolve(c), (uint16_t*)lk.resolve(c),
                         (uint16_t*)lv.resolve(c), B, n_q, n_kv, D, T, theta, eps, c.stream, gp);
        };
        break;
      }
      case TB200_OP_ATTN_DECODE: {
        const int n_q = op.i0, n_kv = op.i1, D = op.i2, window = op.i3;
        // in2 = K cache, weights = V cache (a state tensor id, not a constant)
        if (!b.is_t(op.in0, TB200_BF16, 2) || !b.is_t(op.in1, TB200_I32, 1) || !b.is_t(op.in2, TB200_BF16, 3) ||
            !b.is_t(op.weights, TB200_BF16, 3) || !b.is_t(op.out0, TB200_BF16, 2))
          return b.fail(TB200_INVALID_ARGUMENT, "op %d: attn_decode wants bf16 q [B,q*D], i32 pos, bf16 K/V caches", i);
        if (n_kv != 1 || D != 256 || n_q < 1 || n_q > 4)
          return b.fail(TB200_UNIMPLEMENTED, "op %d: attn_decode supports one KV head of 256 dims and up to 4 query heads", i);
        const int B = tensors[op.in0].shape[0], T = tensors[op.in2].shape[1];
        if (tensors[op.in0].shape[1] != n_q * D || b.numel(op.out0) != (size_t)B * n_q * D ||
            tensors[op.in2].shape[0] != B || tensors[op.in2].shape[2] != D || b.numel(op.weights) != b.numel(op.in2))
          return b.fail(TB200_INVALID_ARGUMENT, "op %d: attn_decode shape mismatch", i);
        const int splits = attn_decode_splits(B);
        scratch_need = std::max(scratch_need, attn_decode_scratch_bytes(B, n_q, splits));
        Loc lq = loc(op.in0), lp = loc(op.in1), lk = loc(op.in2), lv = plan.tensor_loc[op.weights], lo = loc(op.out0);
        const float scale = op.f0;
        step.kernel_name = "attn_decode_splitT";
        step.launches = 2;
        step.launch = [=](const ExecContext& c) {
          launch_attn_decode((const uint16_t*)lq.resolve(c), (const int32_t*)lp.resolve(c), (const uint16_t*)lk.resolve(c),
                             (const uint16_t*)lv.resolve(c), (uint16_t*)lo.resolve(c), (float*)c.scratch, B, n_q, T, window,
                             scale, splits, c.stream);
        };
        break;
      }
      case TB200_OP_GEGLU: {
        if (!b.is_t(op.in0, TB200_BF16, 2) || !b.is_t(op.out0, TB200_BF16, 2) ||
            tensors[op.in0].shape[1] != 2 * tensors[op.out0].shape[1] || tensors[op.in0].shape[0] != tensors[op.out0].shape[0])
          return b.fail(TB200_INVALID_ARGUMENT, "op %d: geglu wants bf16 [B,2I] -> bf16 [B,I]", i);
        const int B = tensors[op.out0].shape[0], I = tensors[op.out0].shape[1];
        Loc lx = loc(op.in0), lo = loc(op.out0);
        const DeferredGemv dg = partials_of(i);
        step.kernel_name = dg.splits > 0 ? "geglu_from_partials" : "geglu";
        step.launch = [=](const ExecContext& c) {
          const GemvPartials gp{dg.splits > 0 ? (const float*)c.scratch : nullptr,
                                dg.splits > 0 ? (const uint16_t*)(c.consts + dg.scale_off) : nullptr, dg.splits};
          launch_geglu((const uint16_t*)lx.resolve(c), (uint16_t*)lo.resolve(c), B, I, c.stream, gp);
        };
        break;
      }
      case TB200_OP_ARGMAX: {
        if ((!b.is_t(op.in0, TB200_BF16, 2) && !b.is_t(op.in0, TB200_F32, 2)) || !b.is_t(op.out0, TB200_I32, 1) ||
            tensors[op.out0].shape[0] != tensors[op.in0].shape[0])
          return b.fail(TB200_INVALID_ARGUMENT, "op %d: argmax wants bf16 or f32 [B,V] -> i32 [B]", i);
        const int is_f32 = tensors[op.in0].dtype == TB200_F32;
        const int B = tensors[op.in0].shape[0], V = tensors[op.in0].shape[1];
        if (op.i1 > 1) needs_fusion = true;  // arg max over the shards of a tensor-parallel group
        scratch_need = std::max(scratch_need, argmax_scratch_bytes(B));
        Loc lx = loc(op.in0), lo = loc(op.out0);
        step.kernel_name = "argmax";
        step.launches = 2;
        step.launch = [=](const ExecContext& c) {
          launch_argmax(lx.resolve(c), is_f32, (int32_t*)lo.resolve(c), c.scratch, B, V, c.stream);
        };
        break;
      }
      case TB200_OP_GEMV_Q8B: {
        if (!b.is_t(op.in0, TB200_BF16, 2) || !b.is_t(op.out0, TB200_BF16, 2) || !b.valid_id(op.weights) ||
            tensors[op.weights].rank != 2 || tensors[op.weights].dtype != TB200_I8)
          return b.fail(TB200_INVALID_ARGUMENT, "op %d: gemv_q8b wants bf16 [B,K] x int8 [K,N] -> bf16 [B,N]", i);
        const int B = tensors[op.in0].shape[0], K = tensors[op.in0].shape[1], N = tensors[op.weights].shape[1], bs = op.i0;
        if (tensors[op.weights].shape[0] != K || tensors[op.out0].shape[0] != B || tensors[op.out0].shape[1] != N)
          return b.fail(TB200_INVALID_ARGUMENT, "op %d: gemv_q8b shape mismatch", i);
        if (bs < 16 || bs % 16 != 0 || K % bs != 0 || K % 16 != 0 || B > 32 || (B > 8 && K % 64 != 0))
          return b.fail(TB200_UNIMPLEMENTED,
                        "op %d: gemv_q8b needs a block size that is a multiple of 16 and divides K, batch <= 8 (<= 32 when K is a multiple of 64)", i);
        const int nblk = K / bs;
        const int8_t* w = b.const_data<int8_t>(op.weights, (size_t)K * N, "weights", i);
        const uint16_t* sc = b.const_data<uint16_t>(op.bias, (size_t)nblk * N, "block scales", i);
        if (!w || !sc) return b.status;
        const int8_t* zp = nullptr;
        if (op.multiplier >= 0 && !(zp = b.const_data<int8_t>(op.multiplier, (size_t)nblk * N, "block zero points", i)))
          return b.status;
        // row-major per output: W^T [N, K], tables [N, K / bs]
        std::vector<int8_t> wt((size_t)N * K), zt(zp ? (size_t)N * nblk : 0);
        std::vector<uint16_t> st((size_t)N * nblk);
        for (int k = 0; k < K; k++)
          for (int nn = 0; nn < N; nn++) wt[(size_t)nn * K + k] = w[(size_t)k * N + nn];
        for (int q = 0; q < nblk; q++)
          for (int nn = 0; nn < N; nn++) {
            st[(size_t)nn * nblk + q] = sc[(size_t)q * N + nn];
            if (zp) zt[(size_t)nn * nblk + q] = zp[(size_t)q * N + nn];
          }
        const size_t w_off = b.add_const(wt.data(), wt.size());
        const size_t s_off = b.add_const(st.data(), st.size() * 2);
        const size_t z_off = zp ? b.add_const(zt.data(), zt.size()) : 0;
        const bool has_zp = zp != nullptr;
        Loc lx = loc(op.in0), lo = loc(op.out0);
        step.kernel_name = "gemv_q8b";
        step.launch = [=](const ExecContext& c) {
          launch_gemv_q8b((const uint16_t*)lx.resolve(c), (const int8_t*)(c.consts + w_off), (const uint16_t*)(c.consts + s_off),
                          has_zp ? (const int8_t*)(c.consts + z_off) : nullptr, (uint16_t*)lo.resolve(c), B, N, K, bs, c.stream);
        };
        break;
      }
      case TB200_OP_ACT_BF16: {
        if (!b.valid_id(op.in0) || !b.valid_id(op.out0) || tensors[op.in0].dtype != TB200_BF16 ||
            tensors[op.out0].dtype != TB200_BF16 || b.numel(op.in0) != b.numel(op.out0) || op.i0 < 0 || op.i0 > 4)
          return b.fail(TB200_INVALID_ARGUMENT, "op %d: act_bf16 wants bf16 tensors of equal size and a function id 0..4", i);
        const long long n = (long long)b.numel(op.in0);
        const int fn = op.i0;
        Loc lx = loc(op.in0), lo = loc(op.out0);
        step.kernel_name = "act_bf16";
        step.launch = [=](const ExecContext& c) {
          launch_act_bf16((const uint16_t*)lx.resolve(c), (uint16_t*)lo.resolve(c), n, fn, c.stream);
        };
        break;
      }
      case TB200_OP_ALLREDUCE: {
        // Only meaningful inside the fused decode step (the exchange happens in that kernel).
        if (!b.is_t(op.in0, TB200_F32, 2) || !b.is_t(op.out0, TB200_BF16, 2) || b.numel(op.in0) != b.numel(op.out0) ||
            op.i0 < 2 || op.i0 > 8 || op.i1 < 0 || op.i1 >= op.i0)
          return b.fail(TB200_INVALID_ARGUMENT, "op %d: allreduce wants f32 [B,H] -> bf16 [B,H], group size 2..8, a rank inside it", i);
        needs_fusion = true;
        step.kernel_name = "allreduce";
        step.launch = [](const ExecContext&) {};
        break;
      }
      case TB200_OP_EW: {
        const bool binary = op.in1 >= 0;
        if (!b.valid_id(op.in0) || !b.valid_id(op.out0) || (binary && !b.valid_id(op.in1)))
          return b.fail(TB200_INVALID_ARGUMENT, "op %d: bad tensor id", i);
        const auto& ta = tensors[op.in0]; const auto& to = tensors[op.out0];
        const tb200_tensor_t* tb = binary ? &tensors[op.in1] : nullptr;
        if (ta.dtype == TB200_I64 || to.dtype == TB200_I64 || (tb && tb->dtype == TB200_I64) || ta.rank != to.rank ||
            (tb && tb->rank != to.rank))
          return b.fail(TB200_INVALID_ARGUMENT, "op %d: elementwise op wants i8/i16/i32/f32/bf16 tensors of equal rank", i);
        EwArgs a{};
        if (op.i0 >= TB200_EW_EXP && op.i0 <= TB200_EW_ERF &&
            (tensors[op.in0].dtype != TB200_F32 && tensors[op.in0].dtype != TB200_BF16))
          return b.fail(TB200_INVALID_ARGUMENT, "op %d: exp / log / reciprocal / rsqrt / tanh / sigmoid / erf want a float tensor", i);
        a.n = (long long)b.numel(op.out0); a.fn = op.i0; a.arg = op.i1;
        a.a_dtype = ta.dtype; a.b_dtype = tb ? tb->dtype : ta.dtype; a.out_dtype = to.dtype;
        a.in_zp = op.in0_zp; a.out_zp = op.out_zp; a.clamp_min = op.clamp_min; a.clamp_max = op.clamp_max;
        a.fmin = op.f0; a.fmax = op.f1; a.bool_result = (op.flags & TB200_FLAG_BOOL_RESULT) ? 1 : 0;
        a.contiguous = 1;
        const int r = (int)to.rank;
        for (int d = 0; d < 4; d++) { a.dims[d] = 1; a.a_str[d] = a.b_str[d] = 0; }
        long long sa = 1, sb = 1;
        for (int d = r - 1; d >= 0; d--) {
          const int od = to.shape[d], ad = ta.shape[d], bd = tb ? tb->shape[d] : od;
          if ((ad != od && ad != 1) || (bd != od && bd != 1))
            return b.fail(TB200_INVALID_ARGUMENT, "op %d: operand shapes do not broadcast to the result", i);
          a.dims[4 - r + d] = od;
          a.a_str[4 - r + d] = ad == 1 && od != 1 ? 0 : (int)sa;
          a.b_str[4 - r + d] = bd == 1 && od != 1 ? 0 : (int)sb;
          if ((ad == 1 && od != 1) || (bd == 1 && od != 1)) a.contiguous = 0;
          sa *= ad; sb *= bd;
        }
        Loc la = loc(op.in0), lb = binary ? loc(op.in1) : Loc{}, lo = loc(op.out0);
        step.kernel_name = "ew";
        step.launch = [=](const ExecContext& c) {
          EwArgs k = a;
          k.a = la.resolve(c); k.b = binary ? lb.resolve(c) : nullptr; k.out = lo.resolve(c);
          launch_ew(k, c.stream);
        };
        break;
      }
      case TB200_OP_TRANSPOSE:
      case TB200_OP_SLICE:
      case TB200_OP_PAD:
      case TB200_OP_CONCAT_AXIS: {
        const bool concat = op.kind == TB200_OP_CONCAT_AXIS;
        if (!b.valid_id(op.in0) || !b.valid_id(op.out0) || (concat && !b.valid_id(op.in1)))
          return b.fail(TB200_INVALID_ARGUMENT, "op %d: bad tensor id", i);
        const auto& ti = tensors[op.in0]; const auto& to = tensors[op.out0];
        const int esz = (int)bytes_of(op.in0) / (int)std::max<size_t>(1, b.numel(op.in0));
        if (ti.dtype != to.dtype || ti.rank != to.rank || (esz != 1 && esz != 2 && esz != 4))
          return b.fail(TB200_INVALID_ARGUMENT, "op %d: wants tensors of one element type (1, 2 or 4 bytes) and equal rank", i);
        const int r = (int)ti.rank;
        const int arg[4] = {op.i0, op.i1, op.i2, op.i3};
        // strides (elements) of a dense tensor, dimensions right-aligned in 6 slots
        auto dense = [&](const tb200_tensor_t& t, long long (&str)[6], int (&dims)[6]) {
          for (int d = 0; d < 6; d++) { str[d] = 0; dims[d] = 1; }
          long long s2 = 1;
          for (int d = (int)t.rank - 1; d >= 0; d--) { str[6 - t.rank + d] = s2; dims[6 - t.rank + d] = t.shape[d]; s2 *= t.shape[d]; }
        };
        std::vector<StridedCopyArgs> parts;
        StridedCopyArgs a{};
        a.elem_bytes = esz; a.pad_elem_bytes = esz; a.pad_value = op.pad_value;
        long long istr[6], ostr[6];
        int idims[6], odims[6];
        dense(ti, istr, idims);
        dense(to, ostr, odims);
        for (int d = 0; d < 6; d++) { a.lo[d] = 0; a.in_dims[d] = 1 << 30; a.out_str[d] = ostr[d]; a.dims[d] = odims[d]; a.in_str[d] = 0; }
        const int o = 6 - r;  // first used slot
        if (op.kind == TB200_OP_TRANSPOSE) {
          bool seen[4] = {false, false, false, false};
          for (int d = 0; d < r; d++) {
            if (arg[d] < 0 || arg[d] >= r || seen[arg[d]] || to.shape[d] != ti.shape[arg[d]])
              return b.fail(TB200_INVALID_ARGUMENT, "op %d: transpose permutation does not match the shapes", i);
            seen[arg[d]] = true;
            a.in_str[o + d] = istr[o + arg[d]];
          }
          parts.push_back(a);
        } else if (op.kind == TB200_OP_SLICE) {
          for (int d = 0; d < r; d++) {
            if (arg[d] < 0 || arg[d] + to.shape[d] > ti.shape[d])
              return b.fail(TB200_INVALID_ARGUMENT, "op %d: slice outside the tensor", i);
            a.in_str[o + d] = istr[o + d];
            a.in_offset += (long long)arg[d] * istr[o + d];
          }
          parts.push_back(a);
        } else if (op.kind == TB200_OP_PAD) {
          for (int d = 0; d < r; d++) {
            if (arg[d] < 0 || arg[d] + ti.shape[d] > to.shape[d])
              return b.fail(TB200_INVALID_ARGUMENT, "op %d: pad amounts do not match the shapes", i);
            a.in_str[o + d] = istr[o + d];
            a.lo[o + d] = arg[d];
            a.in_dims[o + d] = ti.shape[d];
          }
          parts.push_back(a);
        } else {
          const auto& t1 = tensors[op.in1];
          const int axis = op.i0;
          if (axis < 0 || axis >= r || t1.dtype != ti.dtype || t1.rank != ti.rank || ti.shape[axis] + t1.shape[axis] != to.shape[axis])
            return b.fail(TB200_INVALID_ARGUMENT, "op %d: concat shapes do not match", i);
          for (int which = 0; which < 2; which++) {
            const auto& t = which ? t1 : ti;
            StridedCopyArgs c2 = a;
            long long s1[6];
            int d1[6];
            dense(t, s1, d1);
            for (int d = 0; d < 6; d++) { c2.in_str[d] = s1[d]; c2.dims[d] = d1[d]; }
            c2.out_offset = which ? (long long)ti.shape[axis] * ostr[o + axis] : 0;
            parts.push_back(c2);
          }
        }
        for (auto& pt : parts) { pt.n = 1; for (int d = 0; d < 6; d++) pt.n *= pt.dims[d]; widen_strided_copy(pt); }
        Loc l0 = loc(op.in0), l1 = concat ? loc(op.in1) : Loc{}, lo = loc(op.out0);
        step.kernel_name = op.kind == TB200_OP_TRANSPOSE ? "transpose" : op.kind == TB200_OP_SLICE ? "slice"
                           : op.kind == TB200_OP_PAD ? "pad" : "concat_axis";
        step.launches = (int)parts.size();
        step.launch = [=](const ExecContext& c) {
          for (size_t q = 0; q < parts.size(); q++) {
            StridedCopyArgs k = parts[q];
            k.in = (q == 1 ? l1 : l0).resolve(c);
            k.out = lo.resolve(c);
            launch_strided_copy(k, c.stream);
          }
        };
        break;
      }
      case TB200_OP_MATMUL_F: {
        if (!b.valid_id(op.in0) || !b.valid_id(op.in1) || !b.valid_id(op.out0)) return b.fail(TB200_INVALID_ARGUMENT, "op %d: bad tensor id", i);
        const auto& ta = tensors[op.in0]; const auto& tb = tensors[op.in1]; const auto& to = tensors[op.out0];
        const bool in_ok = ta.dtype == TB200_BF16 || ta.dtype == TB200_F32, out_ok = to.dtype == TB200_BF16 || to.dtype == TB200_F32;
        if (!in_ok || !out_ok || tb.dtype != ta.dtype || ta.rank != 2 || tb.rank != 2 || to.rank != 2 || tb.shape[0] != ta.shape[1] ||
            to.shape[0] != ta.shape[0] || to.shape[1] != tb.shape[1])
          return b.fail(TB200_INVALID_ARGUMENT, "op %d: matmul_f wants [M, K] x [K, N] of bf16 or f32 -> [M, N] of f32 or bf16", i);
        const int M = ta.shape[0], K = ta.shape[1], N = tb.shape[1], idt = (int)ta.dtype, odt = (int)to.dtype;
        Loc la = loc(op.in0), lb = loc(op.in1), lo = loc(op.out0);
        step.kernel_name = "matmul_f";
        step.launch = [=](const ExecContext& c) { launch_matmul_f(la.resolve(c), lb.resolve(c), lo.resolve(c), M, K, N, idt, odt, c.stream); };
        break;
      }
      case TB200_OP_DEPTHWISE_F: {
        if (!b.valid_id(op.in0) || !b.valid_id(op.in1) || !b.valid_id(op.in2) || !b.valid_id(op.out0))
          return b.fail(TB200_INVALID_ARGUMENT, "op %d: bad tensor id", i);
        const auto& tx = tensors[op.in0]; const auto& tw = tensors[op.in1]; const auto& tb = tensors[op.in2]; const auto& to = tensors[op.out0];
        DepthwiseFArgs a{};
        a.dtype = (int)tx.dtype;
        if ((tx.dtype != TB200_BF16 && tx.dtype != TB200_F32) || tw.dtype != tx.dtype || tb.dtype != tx.dtype || to.dtype != tx.dtype ||
            tx.rank != 4 || tw.rank != 4 || to.rank != 4 || tw.shape[2] != tx.shape[3] || op.stride_h < 1 || op.stride_w < 1 ||
            op.dil_h < 1 || op.dil_w < 1 || op.pad_t < 0 || op.pad_b < 0 || op.pad_l < 0 || op.pad_r < 0)
          return b.fail(TB200_INVALID_ARGUMENT, "op %d: depthwise_f wants bf16 or f32 x [N,H,W,C], weights [KH,KW,C,M], bias [C*M]", i);
        a.N = tx.shape[0]; a.H = tx.shape[1]; a.W = tx.shape[2]; a.C = tx.shape[3];
        a.KH = tw.shape[0]; a.KW = tw.shape[1]; a.M = tw.shape[3];
        a.stride_h = op.stride_h; a.stride_w = op.stride_w; a.dil_h = op.dil_h; a.dil_w = op.dil_w; a.pad_t = op.pad_t; a.pad_l = op.pad_l;
        a.OH = conv_out_dim(a.H, a.KH, op.stride_h, op.dil_h, op.pad_t, op.pad_b);
        a.OW = conv_out_dim(a.W, a.KW, op.stride_w, op.dil_w, op.pad_l, op.pad_r);
        if (b.numel(op.in2) != (size_t)a.C * a.M || to.shape[0] != a.N || to.shape[1] != a.OH || to.shape[2] != a.OW ||
            to.shape[3] != a.C * a.M)
          return b.fail(TB200_INVALID_ARGUMENT, "op %d: depthwise_f output shape is not %dx%dx%dx%d", i, a.N, a.OH, a.OW, a.C * a.M);
        Loc lx = loc(op.in0), lw = loc(op.in1), lb = loc(op.in2), lo = loc(op.out0);
        step.kernel_name = "depthwise_f";
        step.launch = [=](const ExecContext& c) {
          DepthwiseFArgs k = a;
          k.x = lx.resolve(c); k.w = lw.resolve(c); k.bias = lb.resolve(c); k.out = lo.resolve(c);
          launch_depthwise_f(k, c.stream);
        };
        break;
      }
      case TB200_OP_GATHER:
      case TB200_OP_SCATTER: {
        const bool sc = op.kind == TB200_OP_SCATTER;
        if (!b.valid_id(op.in0) || !b.valid_id(op.in1) || !b.valid_id(op.out0) || (sc && !b.valid_id(op.in2)))
          return b.fail(TB200_INVALID_ARGUMENT, "op %d: bad tensor id", i);
        const auto& tv = tensors[op.in0]; const auto& tix = tensors[op.in1]; const auto& to = tensors[op.out0];
        if (tv.rank != 3 || tix.rank != 2 || tix.dtype != TB200_I32 || to.rank != 3 || to.dtype != tv.dtype || tix.shape[0] != tv.shape[0])
          return b.fail(TB200_INVALID_ARGUMENT, "op %d: wants values [N, K, C], i32 indices [N, W] and a result of the values' type", i);
        const int N = tv.shape[0], K = tv.shape[1], Cc = tv.shape[2], W = tix.shape[1];
        const int esz = (int)bytes_of(op.in0) / (int)std::max<size_t>(1, b.numel(op.in0));
        const int row_bytes = Cc * esz;
        if (sc) {
          const auto& tu = tensors[op.in2];
          if (tu.rank != 3 || tu.dtype != tv.dtype || tu.shape[0] != N || tu.shape[1] != W || tu.shape[2] != Cc || to.shape[0] != N ||
              to.shape[1] != K || to.shape[2] != Cc)
            return b.fail(TB200_INVALID_ARGUMENT, "op %d: scatter wants updates [N, W, C] and a result shaped like the values", i);
        } else if (to.shape[0] != N || to.shape[1] != W || to.shape[2] != Cc) {
          return b.fail(TB200_INVALID_ARGUMENT, "op %d: gather result is not [N, W, C]", i);
        }
        Loc lv = loc(op.in0), li = loc(op.in1), lu = sc ? loc(op.in2) : Loc{}, lo = loc(op.out0);
        const size_t value_bytes = bytes_of(op.in0);
        step.kernel_name = sc ? "scatter" : "gather";
        step.launches = sc ? 2 : 1;
        step.launch = [=](const ExecContext& c) {
          if (sc) {
            cudaMemcpyAsync(lo.resolve(c), lv.resolve(c), value_bytes, cudaMemcpyDeviceToDevice, c.stream);
            launch_scatter_rows(lu.resolve(c), (const int32_t*)li.resolve(c), lo.resolve(c), N, K, W, row_bytes, c.stream);
          } else {
            launch_gather_rows(lv.resolve(c), (const int32_t*)li.resolve(c), lo.resolve(c), N, K, W, row_bytes, c.stream);
          }
        };
        break;
      }
      case TB200_OP_PERMUTE: {
        if (!b.valid_id(op.in0) || !b.valid_id(op.out0) || tensors[op.in0].dtype != tensors[op.out0].dtype ||
            b.numel(op.in0) != b.numel(op.out0))
          return b.fail(TB200_INVALID_ARGUMENT, "op %d: permute wants input and output of the same type and element count", i);
        const int r = (op.i3 >> 24) & 15;
        const int d6[6] = {op.i0 & 0xffff, (op.i0 >> 16) & 0xffff, op.i1 & 0xffff, (op.i1 >> 16) & 0xffff, op.i2 & 0xffff,
                           (op.i2 >> 16) & 0xffff};
        if (r < 1 || r > 6) return b.fail(TB200_INVALID_ARGUMENT, "op %d: permute rank %d outside 1..6", i, r);
        long long in_str[6], total = 1;
        for (int d = r - 1; d >= 0; d--) { in_str[d] = total; total *= d6[d]; }
        bool seen[6] = {false, false, false, false, false, false};
        long long odim[6], ostr_in[6];  // output dimensions in order, each with the input stride it walks
        for (int d = 0; d < r; d++) {
          const int pd = (op.i3 >> (4 * d)) & 15;
          if (pd >= r || seen[pd] || d6[pd] < 1) return b.fail(TB200_INVALID_ARGUMENT, "op %d: bad permutation or extent", i);
          seen[pd] = true;
          odim[d] = d6[pd];
          ostr_in[d] = in_str[pd];
        }
        if ((size_t)total != b.numel(op.in0)) return b.fail(TB200_INVALID_ARGUMENT, "op %d: permute view does not match the tensor", i);
        // drop extents of 1, then merge neighbours that are also neighbours in the input
        int m = 0;
        for (int d = 0; d < r; d++) {
          if (odim[d] == 1) continue;
          if (m > 0 && ostr_in[m - 1] == ostr_in[d] * odim[d]) {
            odim[m - 1] *= odim[d];
            ostr_in[m - 1] = ostr_in[d];
          } else {
            odim[m] = odim[d];
            ostr_in[m] = ostr_in[d];
            m++;
          }
        }
        if (m == 0) { odim[0] = 1; ostr_in[0] = 1; m = 1; }

        StridedCopyArgs a{};
        const int esz = (int)bytes_of(op.in0) / (int)std::max<size_t>(1, b.numel(op.in0));
        if (esz != 1 && esz != 2 && esz != 4) return b.fail(TB200_INVALID_ARGUMENT, "op %d: permute wants 1-, 2- or 4-byte elements", i);
        a.elem_bytes = esz; a.pad_elem_bytes = esz;
        long long ostr = 1;
        for (int d = 0; d < 6; d++) { a.dims[d] = 1; a.lo[d] = 0; a.in_dims[d] = 1 << 30; a.in_str[d] = 0; a.out_str[d] = 0; }
        for (int d = m - 1; d >= 0; d--) {
          const int slot = 6 - m + d;
          if (odim[d] > INT32_MAX) return b.fail(TB200_UNIMPLEMENTED, "op %d: permute extent too large", i);
          a.dims[slot] = (int)odim[d];
          a.in_str[slot] = ostr_in[d];
          a.out_str[slot] = ostr;
          ostr *= odim[d];
        }
        a.n = total;
        widen_strided_copy(a);
        Loc lx = loc(op.in0), lo = loc(op.out0);
        step.kernel_name = "transpose";
        step.launch = [=](const ExecContext& c) {
          StridedCopyArgs k = a;
          k.in = lx.resolve(c);
          k.out = lo.resolve(c);
          launch_strided_copy(k, c.stream);
        };
        break;
      }
      case TB200_OP_SOFTMAX: {
        if (!b.valid_id(op.in0) || !b.valid_id(op.out0) || tensors[op.in0].dtype != tensors[op.out0].dtype ||
            (tensors[op.in0].dtype != TB200_BF16 && tensors[op.in0].dtype != TB200_F32) || b.numel(op.in0) != b.numel(op.out0))
          return b.fail(TB200_INVALID_ARGUMENT, "op %d: softmax wants bf16 or f32 tensors of equal size", i);
        const auto& x = tensors[op.in0];
        const int cols = x.shape[x.rank - 1], dt = (int)x.dtype;
        const long long rows = (long long)(b.numel(op.in0) / cols);
        Loc lx = loc(op.in0), lo = loc(op.out0);
        step.kernel_name = "softmax";
        step.launch = [=](const ExecContext& c) { launch_softmax(lx.resolve(c), lo.resolve(c), rows, cols, dt, c.stream); };
        break;
      }
      case TB200_OP_TABLE16: {
        if (!b.valid_id(op.in0) || !b.valid_id(op.out0) || tensors[op.in0].dtype != TB200_I16 ||
            tensors[op.out0].dtype != TB200_I32 || b.numel(op.in0) != b.numel(op.out0))
          return b.fail(TB200_INVALID_ARGUMENT, "op %d: table16 wants an int16 input and an int32 output of equal size", i);
        const int16_t* tbl = b.const_data<int16_t>(op.table, 513, "table", i);
        if (!tbl) return b.status;
        const size_t t_off = b.add_const(tbl, 513 * 2);
        const long long n = (long long)b.numel(op.in0);
        Loc lx = loc(op.in0), lo = loc(op.out0);
        step.kernel_name = "table16";
        step.launch = [=](const ExecContext& c) {
          launch_table16((const int16_t*)lx.resolve(c), (const int16_t*)(c.consts + t_off), (int32_t*)lo.resolve(c), n, c.stream);
        };
        break;
      }
      case TB200_OP_REDUCE: {
        if (!b.valid_id(op.in0) || !b.valid_id(op.out0)) return b.fail(TB200_INVALID_ARGUMENT, "op %d: bad tensor id", i);
        const auto& ti = tensors[op.in0];
        const int axis = op.i1;
        const bool in_float = ti.dtype == TB200_F32 || ti.dtype == TB200_BF16;
        if (axis < 0 || axis >= (int)ti.rank || op.i0 < 0 || op.i0 > 4 || ti.dtype == TB200_I64 || (op.i0 == 4 && !in_float))
          return b.fail(TB200_INVALID_ARGUMENT, "op %d: bad reduction axis, function or element type", i);
        ReduceArgs a{};
        a.outer = a.inner = 1;
        for (int d = 0; d < axis; d++) a.outer *= ti.shape[d];
        for (int d = axis + 1; d < (int)ti.rank; d++) a.inner *= ti.shape[d];
        a.axis = ti.shape[axis]; a.fn = op.i0; a.in_dtype = ti.dtype; a.out_dtype = tensors[op.out0].dtype;
        if (b.numel(op.out0) != (size_t)a.outer * a.inner)
          return b.fail(TB200_INVALID_ARGUMENT, "op %d: reduction result has the wrong element count", i);
        Loc lx = loc(op.in0), lo = loc(op.out0);
        step.kernel_name = "reduce";
        step.launch = [=](const ExecContext& c) {
          ReduceArgs k = a;
          k.x = lx.resolve(c); k.out = lo.resolve(c);
          launch_reduce(k, c.stream);
        };
        break;
      }
      case TB200_OP_RESHAPE: {
        if (bytes_of(op.in0) != bytes_of(op.out0) || tensors[op.in0].dtype != tensors[op.out0].dtype)
          return b.fail(TB200_INVALID_ARGUMENT, "op %d: reshape changes the byte count", i);
        if (tensors[op.out0].kind == TB200_TENSOR_OUTPUT) {
          const size_t nbytes = bytes_of(op.in0);
          Loc lx = loc(op.in0), lo = loc(op.out0);
          step.kernel_name = "copy (reshape into an output)";
          step.launch = [=](const ExecContext& c) {
            const cudaError_t e = cudaMemcpyAsync(lo.resolve(c), lx.resolve(c), nbytes, cudaMemcpyDeviceToDevice, c.stream);
            if (e != cudaSuccess && c.launch_error) *c.launch_error = e;
          };
          break;
        }
        step.kernel_name = "view";
        step.launches = 0;
        step.launch = [](const ExecContext&) {};
        break;
      }
      default:
        return b.fail(TB200_UNIMPLEMENTED, "op %d: kind %u is not implemented", i, op.kind);
    }
    plan.launch_count += step.launches;
    plan.steps.push_back(std::move(step));
  }
  const bool fused = try_fuse_decode_step(b, plan, scratch_need);
  if (b.status != TB200_OK) return b.status;
  if (needs_fusion && !fused)
    return b.fail(TB200_UNIMPLEMENTED, "tensor-parallel ops run only inside the fused decode step, and this graph does not fit it");
  // scratch shared by the ops that need one, behind the activations
  plan.scratch_offset = (plan.arena_bytes + 255) & ~(size_t)255;
  plan.scratch_bytes = scratch_need;
  plan.arena_bytes = plan.scratch_offset + scratch_need;
  return TB200_OK;
}

}  // namespace tb200
