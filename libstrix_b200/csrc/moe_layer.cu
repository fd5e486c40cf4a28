// Whole-layer launchers: one C call enqueues every kernel of an MoE layer, so a
// host pays one foreign-function call instead of seven and the GPU sees the
// launches back to back. The sequence is the reference's StrixFp8Experts.apply
// (python/strix_vllm/moe.py:905-1014) - permute, quantise, gate-up GEMM with the
// fused gate, quantise, down GEMM x routing weight, sum - preceded by the router
// when logits are given, over the sorted-layout tcgen05 kernels of this library.
// The intermediates live in a caller-provided workspace; nothing is allocated and
// nothing synchronises.
#include "common.cuh"

namespace strix {
namespace {

struct Fp8LayerPlan {
  int64_t cap;                 // sorted rows (capacity of the padded id list)
  int64_t off_ids, off_wts, off_sorted, off_expert, off_post, off_pos;
  int64_t off_xq, off_xs, off_act, off_aq, off_as, off_y, bytes;
};

int64_t up(int64_t x) { return (x + 255) / 256 * 256; }

Fp8LayerPlan plan_fp8(int64_t tokens, int64_t top_k, int64_t hidden, int64_t inter, int64_t experts,
                      int64_t block_m) {
  Fp8LayerPlan p;
  const int64_t slots = tokens * top_k;
  p.cap = strix_moe_align_capacity(slots, experts, block_m);
  int64_t o = 0;
  auto take = [&](int64_t bytes) { const int64_t at = o; o += up(bytes); return at; };
  p.off_ids = take(slots * 4), p.off_wts = take(slots * 4);
  p.off_sorted = take(p.cap * 4), p.off_expert = take((p.cap / block_m) * 4), p.off_post = take(4);
  p.off_pos = take(slots * 4);
  p.off_xq = take(p.cap * hidden), p.off_xs = take(p.cap * (hidden / 128) * 4);
  p.off_act = take(p.cap * inter * 2);
  p.off_aq = take(p.cap * inter), p.off_as = take(p.cap * (inter / 128) * 4);
  p.off_y = take(slots * hidden * 2);
  p.bytes = o;
  return p;
}

}  // namespace
}  // namespace strix

using namespace strix;

extern "C" int64_t strix_moe_fp8_layer_workspace(int64_t tokens, int64_t top_k, int64_t hidden,
                                                 int64_t inter, int64_t experts, int64_t block_m) {
  if (tokens < 0 || top_k < 1 || hidden < 128 || inter < 128 || experts < 1 || block_m < 1) return -1;
  return plan_fp8(tokens, top_k, hidden, inter, experts, block_m).bytes;
}

extern "C" int strix_moe_fp8_layer(
    void* out, const void* x, const float* logits, const float* topk_weights, const int32_t* topk_ids,
    const void* w13, const float* w13_scale, const void* w2, const float* w2_scale, void* workspace,
    int64_t workspace_bytes, int64_t tokens, int64_t hidden, int64_t inter, int64_t experts,
    int64_t top_k, int64_t block_m, int64_t x_stride, int64_t logits_stride, int64_t out_stride,
    int64_t w13_stride_e, int64_t w13_stride_n, int64_t s13_stride_e, int64_t s13_stride_n,
    int64_t w2_stride_e, int64_t w2_stride_n, int64_t s2_stride_e, int64_t s2_stride_n,
    int scale_kind, int gate_act, strix_stream_t stream) {
  STRIX_CHECK(out != nullptr && x != nullptr && w13 != nullptr && w2 != nullptr && w13_scale != nullptr &&
                  w2_scale != nullptr, "pointers must not be NULL");
  STRIX_CHECK((logits != nullptr) != (topk_ids != nullptr && topk_weights != nullptr),
              "pass either router logits or (topk_weights, topk_ids)");
  STRIX_CHECK(tokens >= 0 && hidden % 128 == 0 && inter % 128 == 0 && experts >= 1 && top_k >= 1,
              "hidden and inter must be multiples of 128");
  STRIX_CHECK(gate_act == 1 || gate_act == 2, "activation must be silu or gelu_tanh");
  STRIX_CHECK(strix_moe_gemm_fp8_sorted_covers(2 * inter, hidden, block_m, gate_act, scale_kind) &&
                  strix_moe_gemm_fp8_sorted_covers(hidden, inter, block_m, 0, scale_kind),
              "geometry not covered by the sorted-layout kernels");
  if (tokens == 0) return STRIX_OK;
  const Fp8LayerPlan p = plan_fp8(tokens, top_k, hidden, inter, experts, block_m);
  STRIX_CHECK(workspace != nullptr && workspace_bytes >= p.bytes &&
                  reinterpret_cast<uintptr_t>(workspace) % 256 == 0,
              "workspace of %lld bytes (256-byte aligned) required, got %lld", (long long)p.bytes,
              (long long)workspace_bytes);
  uint8_t* ws = static_cast<uint8_t*>(workspace);
  auto i32 = [&](int64_t off) { return reinterpret_cast<int32_t*>(ws + off); };
  auto f32 = [&](int64_t off) { return reinterpret_cast<float*>(ws + off); };
  const int64_t slots = tokens * top_k;
  const int32_t* ids = topk_ids;
  const float* wts = topk_weights;
  int rc;
  if (logits != nullptr) {
    if ((rc = strix_moe_topk_softmax(logits, i32(p.off_ids), f32(p.off_wts), tokens, experts, top_k,
                                     logits_stride, 1, stream)))
      return rc;
    ids = i32(p.off_ids), wts = f32(p.off_wts);
  }
  if ((rc = strix_moe_align_pos(ids, i32(p.off_sorted), i32(p.off_expert), i32(p.off_post),
                                i32(p.off_pos), slots, experts, block_m, p.cap, p.cap / block_m, stream)))
    return rc;
  if ((rc = strix_moe_act_quant_fp8_scatter(x, ws + p.off_xq, f32(p.off_xs), i32(p.off_pos),
                                            i32(p.off_sorted), i32(p.off_post), tokens, p.cap, hidden,
                                            top_k, x_stride, hidden, hidden / 128, 0, stream)))
    return rc;
  if ((rc = strix_moe_gemm_fp8_sorted(ws + p.off_act, ws + p.off_xq, f32(p.off_xs), w13, w13_scale,
                                      i32(p.off_sorted), i32(p.off_expert), i32(p.off_post), nullptr,
                                      slots, experts, 2 * inter, hidden, hidden, inter, w13_stride_e,
                                      w13_stride_n, s13_stride_e, s13_stride_n, hidden / 128, p.cap,
                                      block_m, scale_kind, gate_act, /*c_sorted=*/1, stream)))
    return rc;
  if ((rc = strix_moe_act_quant_fp8_sorted(ws + p.off_act, ws + p.off_aq, f32(p.off_as), nullptr,
                                           i32(p.off_post), p.cap, inter, 1, slots, inter, inter,
                                           inter / 128, 0, stream)))
    return rc;
  if ((rc = strix_moe_gemm_fp8_sorted(ws + p.off_y, ws + p.off_aq, f32(p.off_as), w2, w2_scale,
                                      i32(p.off_sorted), i32(p.off_expert), i32(p.off_post), wts, slots,
                                      experts, hidden, inter, inter, hidden, w2_stride_e, w2_stride_n,
                                      s2_stride_e, s2_stride_n, inter / 128, p.cap, block_m, scale_kind,
                                      /*gate_act=*/0, /*c_sorted=*/0, stream)))
    return rc;
  return strix_moe_sum(ws + p.off_y, out, tokens, top_k, hidden, top_k * hidden, hidden, out_stride, stream);
}
