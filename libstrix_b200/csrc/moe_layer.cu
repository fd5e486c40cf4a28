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
  int64_t off_xq, off_xs, off_act, off_aq, off_as, off_y, off_hist, hist_bytes, bytes;
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
  // wide enough for payload rows too (e4m3 bytes, then the row's scales, 16-byte padded)
  p.off_xq = take(p.cap * ((hidden + hidden / 32 + 15) / 16 * 16));
  p.off_xs = take(p.cap * (hidden / 128) * 4);
  p.off_act = take(p.cap * inter * 2);
  p.off_aq = take(p.cap * inter), p.off_as = take(p.cap * (inter / 128) * 4);
  p.off_y = take(slots * hidden * 2);
  p.hist_bytes = strix_moe_align_scratch_bytes(slots, experts);
  p.off_hist = take(p.hist_bytes);
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

// x_quantised: x is a payload of e4m3 rows followed by their fp32 group scales
// (x_stride in bytes) instead of bf16 rows (x_stride in elements). sum_output 0
// leaves the weighted rows in slot order in `out` ([tokens * top_k, hidden]).
static int fp8_layer_impl(
    void* out, const void* x, const float* logits, const float* topk_weights, const int32_t* topk_ids,
    const void* w13, const float* w13_scale, const void* w2, const float* w2_scale, void* workspace,
    int64_t workspace_bytes, int64_t tokens, int64_t hidden, int64_t inter, int64_t experts,
    int64_t top_k, int64_t block_m, int64_t x_stride, int64_t logits_stride, int64_t out_stride,
    int64_t w13_stride_e, int64_t w13_stride_n, int64_t s13_stride_e, int64_t s13_stride_n,
    int64_t w2_stride_e, int64_t w2_stride_n, int64_t s2_stride_e, int64_t s2_stride_n,
    int scale_kind, int gate_act, int x_quantised, int sum_output, strix_stream_t stream) {
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
  if ((rc = strix_moe_align_scratch(ids, i32(p.off_sorted), i32(p.off_expert), i32(p.off_post),
                                    i32(p.off_pos), nullptr, ws + p.off_hist, p.hist_bytes, slots, experts,
                                    block_m, p.cap, p.cap / block_m, stream)))
    return rc;
  // sorted activations: e4m3 rows [cap, hidden] + scales [cap, hidden / 128], or - for
  // a payload that arrives quantised - whole payload rows, scales behind the bytes
  const uint8_t* xq = ws + p.off_xq;
  const float* xs = f32(p.off_xs);
  int64_t xq_stride = hidden, xs_stride = hidden / 128;
  if (x_quantised) {
    const int64_t row_bytes = (hidden + hidden / 32 + 15) / 16 * 16;
    STRIX_CHECK(x_stride >= row_bytes && x_stride % 16 == 0, "payload rows must be whole 16-byte chunks");
    if ((rc = strix_moe_permute_rows(x, ws + p.off_xq, i32(p.off_pos), i32(p.off_sorted), i32(p.off_post),
                                     tokens, p.cap, row_bytes, top_k, x_stride, row_bytes, stream)))
      return rc;
    xs = reinterpret_cast<const float*>(xq + hidden);
    xq_stride = row_bytes, xs_stride = row_bytes / 4;
  } else if ((rc = strix_moe_act_quant_fp8_scatter(x, ws + p.off_xq, f32(p.off_xs), i32(p.off_pos),
                                                   i32(p.off_sorted), i32(p.off_post), tokens, p.cap,
                                                   hidden, top_k, x_stride, hidden, hidden / 128, 0,
                                                   stream))) {
    return rc;
  }
  if ((rc = strix_moe_gemm_fp8_sorted(ws + p.off_act, xq, xs, w13, w13_scale,
                                      i32(p.off_sorted), i32(p.off_expert), i32(p.off_post), nullptr,
                                      slots, experts, 2 * inter, hidden, xq_stride, inter, w13_stride_e,
                                      w13_stride_n, s13_stride_e, s13_stride_n, xs_stride, p.cap,
                                      block_m, scale_kind, gate_act, /*c_sorted=*/1, stream)))
    return rc;
  if ((rc = strix_moe_act_quant_fp8_sorted(ws + p.off_act, ws + p.off_aq, f32(p.off_as), nullptr,
                                           i32(p.off_post), p.cap, inter, 1, slots, inter, inter,
                                           inter / 128, 0, stream)))
    return rc;
  void* y = sum_output ? static_cast<void*>(ws + p.off_y) : out;
  const int64_t y_stride = sum_output ? hidden : out_stride;
  if ((rc = strix_moe_gemm_fp8_sorted(y, ws + p.off_aq, f32(p.off_as), w2, w2_scale,
                                      i32(p.off_sorted), i32(p.off_expert), i32(p.off_post), wts, slots,
                                      experts, hidden, inter, inter, y_stride, w2_stride_e, w2_stride_n,
                                      s2_stride_e, s2_stride_n, inter / 128, p.cap, block_m, scale_kind,
                                      /*gate_act=*/0, /*c_sorted=*/0, stream)))
    return rc;
  if (!sum_output) return STRIX_OK;
  return strix_moe_sum(ws + p.off_y, out, tokens, top_k, hidden, top_k * hidden, hidden, out_stride, stream);
}

extern "C" int strix_moe_fp8_layer(
    void* out, const void* x, const float* logits, const float* topk_weights, const int32_t* topk_ids,
    const void* w13, const float* w13_scale, const void* w2, const float* w2_scale, void* workspace,
    int64_t workspace_bytes, int64_t tokens, int64_t hidden, int64_t inter, int64_t experts,
    int64_t top_k, int64_t block_m, int64_t x_stride, int64_t logits_stride, int64_t out_stride,
    int64_t w13_stride_e, int64_t w13_stride_n, int64_t s13_stride_e, int64_t s13_stride_n,
    int64_t w2_stride_e, int64_t w2_stride_n, int64_t s2_stride_e, int64_t s2_stride_n,
    int scale_kind, int gate_act, strix_stream_t stream) {
  return fp8_layer_impl(out, x, logits, topk_weights, topk_ids, w13, w13_scale, w2, w2_scale, workspace,
                        workspace_bytes, tokens, hidden, inter, experts, top_k, block_m, x_stride,
                        logits_stride, out_stride, w13_stride_e, w13_stride_n, s13_stride_e, s13_stride_n,
                        w2_stride_e, w2_stride_n, s2_stride_e, s2_stride_n, scale_kind, gate_act, 0, 1,
                        stream);
}

// The experts of the layer over rows that arrive quantised and whose slots may be
// masked (expert id -1): the receiving side of the expert-parallel exchange. rows =
// payload rows [rows, row_stride_bytes] (e4m3 bytes, then fp32 scales per 128), ids /
// weights [rows, top_k]; y receives the weighted result rows in slot order ([rows *
// top_k, hidden], rows of masked slots untouched).
extern "C" int strix_moe_fp8_experts_on_rows(
    void* y, const void* rows_payload, const float* topk_weights, const int32_t* topk_ids,
    const void* w13, const float* w13_scale, const void* w2, const float* w2_scale, void* workspace,
    int64_t workspace_bytes, int64_t rows, int64_t hidden, int64_t inter, int64_t experts,
    int64_t top_k, int64_t block_m, int64_t row_stride_bytes, int64_t y_stride,
    int64_t w13_stride_e, int64_t w13_stride_n, int64_t s13_stride_e, int64_t s13_stride_n,
    int64_t w2_stride_e, int64_t w2_stride_n, int64_t s2_stride_e, int64_t s2_stride_n,
    int scale_kind, int gate_act, strix_stream_t stream) {
  STRIX_CHECK(topk_weights != nullptr && topk_ids != nullptr, "routing must not be NULL");
  return fp8_layer_impl(y, rows_payload, nullptr, topk_weights, topk_ids, w13, w13_scale, w2, w2_scale,
                        workspace, workspace_bytes, rows, hidden, inter, experts, top_k, block_m,
                        row_stride_bytes, 0, y_stride, w13_stride_e, w13_stride_n, s13_stride_e,
                        s13_stride_n, w2_stride_e, w2_stride_n, s2_stride_e, s2_stride_n, scale_kind,
                        gate_act, 1, 0, stream);
}


// ------------------------------------------------------- expert-parallel layer
namespace strix {
namespace {

struct EpLayerPlan {
  int64_t rows, slots, cap;       // received rows (world * exchange capacity), their slots, sorted rows
  int64_t off_ids, off_wts, off_payload;                       // this rank's routing, FP8 payload
  int64_t off_sorted, off_expert, off_post, off_pos, off_xs, off_act, off_hist, hist_bytes;   // MXFP4 receiving side
  int64_t off_inner, inner_bytes;                              // FP8 receiving side (plan_fp8)
  int64_t bytes;
};

EpLayerPlan plan_ep(const strix_expert_weights& w, const strix_ep_exchange& ep, int64_t block_m) {
  EpLayerPlan p{};
  p.rows = ep.world * ep.cap;
  p.slots = p.rows * ep.top_k;
  p.cap = strix_moe_align_capacity(p.slots, w.experts, block_m);
  int64_t o = 0;
  auto take = [&](int64_t bytes) { const int64_t at = o; o += up(bytes); return at; };
  p.off_ids = take(ep.cap * ep.top_k * 4), p.off_wts = take(ep.cap * ep.top_k * 4);
  if (w.kind == 0) {
    p.off_payload = 0;
    p.off_sorted = take(p.cap * 4), p.off_expert = take((p.cap / block_m) * 4), p.off_post = take(4);
    p.off_pos = take(p.slots * 4);
    p.off_xs = take(p.cap * w.hidden * 2), p.off_act = take(p.cap * w.inter * 2);
    p.hist_bytes = strix_moe_align_scratch_bytes(p.slots, w.experts);
    p.off_hist = take(p.hist_bytes);
  } else {
    p.off_payload = take(ep.cap * ep.row_bytes);
    p.inner_bytes = plan_fp8(p.rows, ep.top_k, w.hidden, w.inter, w.experts, block_m).bytes;
    p.off_inner = take(p.inner_bytes);
  }
  p.bytes = o;
  return p;
}

int check_ep(const strix_expert_weights* w, const strix_ep_exchange* ep, int64_t block_m) {
  STRIX_CHECK(w != nullptr && ep != nullptr, "weights and exchange must not be NULL");
  STRIX_CHECK(w->kind >= 0 && w->kind <= 2, "weight kind must be 0 (MXFP4), 1 or 2 (FP8 channel / block scales)");
  STRIX_CHECK(w->experts >= 1 && w->hidden >= 128 && w->inter >= 64, "bad expert geometry");
  STRIX_CHECK(ep->world >= 1 && ep->world <= 16 && ep->rank >= 0 && ep->rank < ep->world && ep->cap >= 1 &&
                  ep->top_k >= 1 && ep->top_k <= 31 && ep->hidden == w->hidden, "bad exchange geometry");
  const int64_t row = w->kind == 0 ? w->hidden * 2 : (w->hidden + w->hidden / 32 + 15) / 16 * 16;
  STRIX_CHECK(ep->row_bytes == row, "the exchange's payload row is %lld bytes, this layer sends %lld",
              (long long)ep->row_bytes, (long long)row);
  STRIX_CHECK(block_m >= 1 && (w->kind != 0 || block_m == 128), "MXFP4 experts take m-blocks of 128");
  return STRIX_OK;
}

}  // namespace
}  // namespace strix

extern "C" int64_t strix_ep_moe_layer_workspace(const strix_expert_weights* w, const strix_ep_exchange* ep,
                                                int64_t block_m) {
  if (check_ep(w, ep, block_m) != STRIX_OK) return -1;
  return plan_ep(*w, *ep, block_m).bytes;
}

// Router -> [quantise] -> plan -> dispatch into the owners' buffers -> wait for the
// sources -> experts over the received rows -> partial sums back to the sources ->
// wait and combine: every kernel of one expert-parallel layer, enqueued by one call.
extern "C" int strix_ep_moe_layer(void* out, const void* x, const float* logits,
                                  const strix_expert_weights* w, const strix_ep_exchange* ep,
                                  void* workspace, int64_t workspace_bytes, int64_t tokens,
                                  int64_t x_stride, int64_t logits_stride, int64_t out_stride,
                                  int64_t block_m, int64_t spin_limit, strix_stream_t stream) {
  if (int rc = check_ep(w, ep, block_m)) return rc;
  STRIX_CHECK(tokens >= 0 && tokens <= ep->cap, "%lld tokens exceed the exchange capacity %lld",
              (long long)tokens, (long long)ep->cap);
  STRIX_CHECK(tokens == 0 || (out != nullptr && x != nullptr && logits != nullptr), "pointers must not be NULL");
  const EpLayerPlan p = plan_ep(*w, *ep, block_m);
  STRIX_CHECK(workspace != nullptr && workspace_bytes >= p.bytes &&
                  reinterpret_cast<uintptr_t>(workspace) % 256 == 0,
              "workspace of %lld bytes (256-byte aligned) required, got %lld", (long long)p.bytes,
              (long long)workspace_bytes);
  uint8_t* ws = static_cast<uint8_t*>(workspace);
  auto i32 = [&](int64_t off) { return reinterpret_cast<int32_t*>(ws + off); };
  auto f32 = [&](int64_t off) { return reinterpret_cast<float*>(ws + off); };
  const int64_t k = ep->top_k, h = w->hidden, inter = w->inter;
  const int64_t epr = ep->round_robin ? -w->experts : w->experts;   // how experts map to ranks
  int rc;
  // ---- this rank's tokens: route, (quantise,) send
  const void* payload = x;
  int64_t payload_stride = x_stride * 2;
  if (tokens > 0) {
    const int64_t e_global = ep->experts_global > 0 ? ep->experts_global : w->experts * ep->world;
    if ((rc = strix_moe_topk_softmax(logits, i32(p.off_ids), f32(p.off_wts), tokens, e_global, k,
                                     logits_stride, 1, stream)))
      return rc;
    if (w->kind != 0) {
      uint8_t* q = ws + p.off_payload;
      if ((rc = strix_moe_act_quant_fp8(x, q, reinterpret_cast<float*>(q + h), tokens, h, x_stride,
                                        ep->row_bytes, ep->row_bytes / 4, 0, stream)))
        return rc;
      payload = q, payload_stride = ep->row_bytes;
    }
  }
  if ((rc = strix_ep_plan(i32(p.off_ids), ep->tok_pos, ep->counts, tokens, k, epr, ep->world, ep->placement,
                          stream)))
    return rc;
  if ((rc = strix_ep_dispatch(payload, i32(p.off_ids), f32(p.off_wts), ep->tok_pos, ep->counts,
                              ep->peer_recv, ep->peer_meta, ep->peer_counts, ep->peer_flags, ep->ticket,
                              tokens, ep->row_bytes, payload_stride, k, epr, ep->world, ep->rank,
                              ep->cap, ep->epoch, ep->placement, stream)))
    return rc;
  // ---- the rows other ranks sent here: through this rank's experts
  const void* recv = ep->peer_recv[ep->rank];
  if ((rc = strix_ep_prepare(static_cast<const int32_t*>(ep->peer_meta[ep->rank]),
                             static_cast<const int32_t*>(ep->peer_counts[ep->rank]),
                             static_cast<const int32_t*>(ep->peer_flags[ep->rank]), ep->ids, ep->weights,
                             ep->rows_per_source, ep->world, ep->cap, k, ep->epoch, spin_limit, stream)))
    return rc;
  if (w->kind == 0) {
    if ((rc = strix_moe_align_scratch(ep->ids, i32(p.off_sorted), i32(p.off_expert), i32(p.off_post),
                                      i32(p.off_pos), nullptr, ws + p.off_hist, p.hist_bytes, p.slots,
                                      w->experts, block_m, p.cap, p.cap / block_m, stream)))
      return rc;
    if ((rc = strix_moe_permute_rows(recv, ws + p.off_xs, i32(p.off_pos), i32(p.off_sorted),
                                     i32(p.off_post), p.rows, p.cap, h * 2, k, ep->row_bytes, h * 2, stream)))
      return rc;
    if ((rc = strix_moe_gemm_mxfp4_sorted(ws + p.off_act, ws + p.off_xs, w->w13, w->w13_scale,
                                          i32(p.off_sorted), i32(p.off_expert), i32(p.off_post), nullptr,
                                          p.slots, w->experts, 2 * inter, h, h, inter, w->w13_stride_e,
                                          w->w13_stride_n, w->s13_stride_e, w->s13_stride_n, p.cap, block_m,
                                          w->gate_act, 1, stream)))
      return rc;
    if ((rc = strix_moe_gemm_mxfp4_sorted(ep->y, ws + p.off_act, w->w2, w->w2_scale, i32(p.off_sorted),
                                          i32(p.off_expert), i32(p.off_post), ep->weights, p.slots,
                                          w->experts, h, inter, inter, h, w->w2_stride_e, w->w2_stride_n,
                                          w->s2_stride_e, w->s2_stride_n, p.cap, block_m, 0, 0, stream)))
      return rc;
  } else {
    if ((rc = fp8_layer_impl(ep->y, recv, nullptr, ep->weights, ep->ids, w->w13,
                             static_cast<const float*>(w->w13_scale), w->w2,
                             static_cast<const float*>(w->w2_scale), ws + p.off_inner, p.inner_bytes, p.rows,
                             h, inter, w->experts, k, block_m, ep->row_bytes, 0, h, w->w13_stride_e,
                             w->w13_stride_n, w->s13_stride_e, w->s13_stride_n, w->w2_stride_e,
                             w->w2_stride_n, w->s2_stride_e, w->s2_stride_n, w->kind, w->gate_act, 1, 0,
                             stream)))
      return rc;
  }
  // ---- partial sums back to their sources, then this rank's own combine
  if ((rc = strix_ep_return(ep->y, ep->ids, static_cast<const int32_t*>(ep->peer_meta[ep->rank]),
                            static_cast<const int32_t*>(ep->peer_counts[ep->rank]), ep->peer_ret,
                            ep->peer_rflags, ep->ticket + 1, ep->world, ep->rank, ep->cap, k, h, h,
                            ep->epoch, stream)))
    return rc;
  return strix_ep_combine(ep->peer_ret[ep->rank], static_cast<const int32_t*>(ep->peer_rflags[ep->rank]),
                          ep->tok_pos, out, tokens, h, tokens ? out_stride : h, ep->world, ep->cap,
                          ep->epoch, spin_limit, stream);
}
