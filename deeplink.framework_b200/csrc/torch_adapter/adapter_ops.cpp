// Operator half of the eager adapter: the aten entries of the transformer-inference path, each calling the DIOPI function
// the reference's generated wrapper calls for it (dipu/scripts/autogen_diopi_wrapper/diopi_functions.yaml, lines cited per
// op). Structured ops are registered through their `.out` overload only: torch's structured wrappers derive the functional
// and in-place forms from it, with output shape, dtype promotion and allocation done by the op's meta function.
#include <cmath>

#include <ATen/ExpandUtils.h>
#include <ATen/WrapDimUtils.h>
#include <ATen/WrapDimUtilsMulti.h>
#include <ATen/native/DispatchStub.h>
#include <ATen/native/transformers/attention.h>
#include <torch/library.h>

#include "adapter_common.h"

namespace dipu_b200 {
namespace {

// A 0-dim host tensor: what a Python number becomes in a binary op (the reference tests is_scalar_on_cpu, yaml:26-38).
bool is_cpu_scalar(const at::Tensor& t) { return t.is_cpu() && t.dim() == 0; }

const at::Tensor& device_of(const at::Tensor& a, const at::Tensor& b) { return a.is_cpu() ? b : a; }

diopiSize_t size_of(c10::IntArrayRef v) {
    diopiSize_t s;
    s.data = v.data();
    s.len = static_cast<int64_t>(v.size());
    return s;
}

// ---- binary arithmetic ------------------------------------------------------------------------------------------------------
// yaml:26-69 (add), 72-92 (sub), 159-202 (mul), 94-151 (div)
at::Tensor& add_out(const at::Tensor& self, const at::Tensor& other, const at::Scalar& alpha, at::Tensor& out) {
    const c10::DeviceGuard guard(out.device());
    CallContext ctx(out);
    Wrapped o(out);
    const diopiScalar_t a = to_diopi_scalar(alpha);
    if (is_cpu_scalar(other) || is_cpu_scalar(self)) {
        // number + tensor = tensor + number; with alpha: self + alpha * other, so a scalar `self` needs the product form
        if (is_cpu_scalar(other)) {
            Wrapped s(self);
            const diopiScalar_t v = to_diopi_scalar(other.item());
            DIPU_B200_CALL(diopiAddScalar(&ctx, &o, &s, &v, &a));
        } else {
            TORCH_CHECK(alpha.toDouble() == 1.0, "add(number, tensor, alpha != 1) is not supported on dipu");
            Wrapped s(other);
            const diopiScalar_t v = to_diopi_scalar(self.item());
            DIPU_B200_CALL(diopiAddScalar(&ctx, &o, &s, &v, &a));
        }
        return out;
    }
    Wrapped s(self), t(other);
    DIPU_B200_CALL(diopiAdd(&ctx, &o, &s, &t, &a));
    return out;
}

at::Tensor& sub_out(const at::Tensor& self, const at::Tensor& other, const at::Scalar& alpha, at::Tensor& out) {
    const c10::DeviceGuard guard(out.device());
    CallContext ctx(out);
    Wrapped o(out);
    const diopiScalar_t a = to_diopi_scalar(alpha);
    TORCH_CHECK(!is_cpu_scalar(self), "sub(number, tensor) is not supported on dipu");
    Wrapped s(self);
    if (is_cpu_scalar(other)) {
        const diopiScalar_t v = to_diopi_scalar(other.item());
        DIPU_B200_CALL(diopiSubScalar(&ctx, &o, &s, &v, &a));
    } else {
        Wrapped t(other);
        DIPU_B200_CALL(diopiSub(&ctx, &o, &s, &t, &a));
    }
    return out;
}

at::Tensor& mul_out(const at::Tensor& self, const at::Tensor& other, at::Tensor& out) {
    const c10::DeviceGuard guard(out.device());
    CallContext ctx(out);
    Wrapped o(out);
    // the CUDA vendor does not divert host scalars for mul (yaml:169-183): the library takes a 0-dim host tensor as `other`
    const at::Tensor& a = is_cpu_scalar(self) ? other : self;
    const at::Tensor& b = is_cpu_scalar(self) ? self : other;
    Wrapped s(a), t(b);
    DIPU_B200_CALL(diopiMul(&ctx, &o, &s, &t));
    return out;
}

at::Tensor& div_out(const at::Tensor& self, const at::Tensor& other, at::Tensor& out) {
    const c10::DeviceGuard guard(out.device());
    CallContext ctx(out);
    Wrapped o(out);
    TORCH_CHECK(!is_cpu_scalar(self), "div(number, tensor) is not supported on dipu");
    Wrapped s(self);
    if (is_cpu_scalar(other)) {
        const diopiScalar_t v = to_diopi_scalar(other.item());
        DIPU_B200_CALL(diopiDivScalar(&ctx, &o, &s, &v, RoundModeNone));
    } else {
        Wrapped t(other);
        DIPU_B200_CALL(diopiDiv(&ctx, &o, &s, &t, RoundModeNone));
    }
    return out;
}

// ---- unary --------------------------------------------------------------------------------------------------------------------
#define DIPU_B200_UNARY(NAME, DIOPI_FN)                                     \
    at::Tensor& NAME(const at::Tensor& self, at::Tensor& out) {             \
        const c10::DeviceGuard guard(out.device());                         \
        CallContext ctx(out);                                               \
        Wrapped o(out), s(self);                                            \
        DIPU_B200_CALL(DIOPI_FN(&ctx, &o, &s));                             \
        return out;                                                         \
    }
DIPU_B200_UNARY(silu_out, diopiSilu)          // yaml:1767-1786
DIPU_B200_UNARY(neg_out, diopiNeg)            // yaml:787-791
DIPU_B200_UNARY(rsqrt_out, diopiRsqrt)        // yaml:1179-1185
DIPU_B200_UNARY(sqrt_out, diopiSqrt)          // yaml:794-802
DIPU_B200_UNARY(reciprocal_out, diopiReciprocal)
DIPU_B200_UNARY(exp_out, diopiExp)
DIPU_B200_UNARY(cos_out, diopiCos)            // yaml:1733-1753
DIPU_B200_UNARY(sin_out, diopiSin)
DIPU_B200_UNARY(sigmoid_out, diopiSigmoid)
DIPU_B200_UNARY(tanh_out, diopiTanh)
#undef DIPU_B200_UNARY

// yaml:1299-1327
at::Tensor& pow_tensor_scalar_out(const at::Tensor& self, const at::Scalar& exponent, at::Tensor& out) {
    const c10::DeviceGuard guard(out.device());
    CallContext ctx(out);
    Wrapped o(out), s(self);
    const diopiScalar_t e = to_diopi_scalar(exponent);
    DIPU_B200_CALL(diopiPow(&ctx, &o, &s, &e));
    return out;
}

// ---- reductions / normalisation ----------------------------------------------------------------------------------------------
// yaml:830-842
at::Tensor& mean_out(const at::Tensor& self, at::OptionalIntArrayRef dim, bool keepdim, std::optional<at::ScalarType> dtype, at::Tensor& out) {
    (void)keepdim;
    (void)dtype;
    const c10::DeviceGuard guard(out.device());
    CallContext ctx(out);
    Wrapped o(out), s(self);
    std::vector<int64_t> dims;
    if (dim.has_value()) {
        for (int64_t d : dim.value()) dims.push_back(at::maybe_wrap_dim(d, self.dim()));
    }
    DIPU_B200_CALL(diopiMean(&ctx, &o, &s, size_of(dims)));
    return out;
}

// yaml:1290-1292
at::Tensor& softmax_out(const at::Tensor& self, int64_t dim, bool half_to_float, at::Tensor& out) {
    (void)half_to_float;  // `out` already has the result dtype
    const c10::DeviceGuard guard(out.device());
    CallContext ctx(out);
    Wrapped o(out), s(self);
    DIPU_B200_CALL(diopiSoftmax(&ctx, &o, &s, at::maybe_wrap_dim(dim, self.dim())));
    return out;
}

// yaml:350-369: mean / rstd take the input dtype and shape [..., 1, ...]; out is contiguous
std::tuple<at::Tensor, at::Tensor, at::Tensor> native_layer_norm(const at::Tensor& input, c10::IntArrayRef normalized_shape,
                                                                const std::optional<at::Tensor>& weight, const std::optional<at::Tensor>& bias, double eps) {
    const c10::DeviceGuard guard(input.device());
    const int64_t lead = input.dim() - static_cast<int64_t>(normalized_shape.size());
    TORCH_CHECK(lead >= 0, "native_layer_norm: normalized_shape has more dimensions than the input");
    std::vector<int64_t> stat_shape(input.sizes().begin(), input.sizes().begin() + lead);
    stat_shape.resize(input.dim(), 1);
    at::Tensor out = at::empty(input.sizes(), input.options());
    at::Tensor mean = at::empty(stat_shape, input.options());
    at::Tensor rstd = at::empty(stat_shape, input.options());
    CallContext ctx(out);
    Wrapped o(out), m(mean), r(rstd), x(input), w, b;
    const bool has_w = weight.has_value() && weight->defined(), has_b = bias.has_value() && bias->defined();
    if (has_w) w = Wrapped(*weight);
    if (has_b) b = Wrapped(*bias);
    DIPU_B200_CALL(diopiLayerNorm(&ctx, &o, &m, &r, &x, has_w ? &w : nullptr, has_b ? &b : nullptr, size_of(normalized_shape), eps));
    return {out, mean, rstd};
}

// aten::_fused_rms_norm (torch >= 2.9): the fused form of the module's pow / mean / rsqrt / mul sequence
std::tuple<at::Tensor, at::Tensor> fused_rms_norm(const at::Tensor& input, c10::IntArrayRef normalized_shape, const std::optional<at::Tensor>& weight,
                                                  std::optional<double> eps) {
    const c10::DeviceGuard guard(input.device());
    const int64_t lead = input.dim() - static_cast<int64_t>(normalized_shape.size());
    TORCH_CHECK(lead >= 0, "_fused_rms_norm: normalized_shape has more dimensions than the input");
    std::vector<int64_t> stat_shape(input.sizes().begin(), input.sizes().begin() + lead);
    stat_shape.resize(input.dim(), 1);
    at::Tensor out = at::empty(input.sizes(), input.options());
    at::Tensor rstd = at::empty(stat_shape, input.options().dtype(at::kFloat));
    const double e = eps.has_value() ? *eps : static_cast<double>(std::numeric_limits<float>::epsilon());
    CallContext ctx(out);
    Wrapped o(out), r(rstd), x(input), w;
    const bool has_w = weight.has_value() && weight->defined();
    if (has_w) w = Wrapped(*weight);
    DIPU_B200_CALL(diopiRMSNorm(&ctx, &o, &r, &x, size_of(normalized_shape), has_w ? &w : nullptr, nullptr, e));
    return {out, rstd};
}

// ---- contractions ---------------------------------------------------------------------------------------------------------------
// yaml:1829-1837 (mm), 1755-1765 (bmm), 594-597 (addmm), 1534-1554 (baddbmm)
at::Tensor& mm_out(const at::Tensor& self, const at::Tensor& mat2, at::Tensor& out) {
    const c10::DeviceGuard guard(out.device());
    CallContext ctx(out);
    Wrapped o(out), a(self), b(mat2);
    DIPU_B200_CALL(diopiMm(&ctx, &o, &a, &b));
    return out;
}

at::Tensor& bmm_out(const at::Tensor& self, const at::Tensor& mat2, at::Tensor& out) {
    const c10::DeviceGuard guard(out.device());
    CallContext ctx(out);
    Wrapped o(out), a(self), b(mat2);
    DIPU_B200_CALL(diopiBmm(&ctx, &o, &a, &b));
    return out;
}

at::Tensor& addmm_out(const at::Tensor& self, const at::Tensor& mat1, const at::Tensor& mat2, const at::Scalar& beta, const at::Scalar& alpha,
                      at::Tensor& out) {
    const c10::DeviceGuard guard(out.device());
    CallContext ctx(out);
    Wrapped o(out), s(self), a(mat1), b(mat2);
    const diopiScalar_t be = to_diopi_scalar(beta), al = to_diopi_scalar(alpha);
    DIPU_B200_CALL(diopiAddmm(&ctx, &o, &s, &a, &b, &be, &al));
    return out;
}

at::Tensor& baddbmm_out(const at::Tensor& self, const at::Tensor& batch1, const at::Tensor& batch2, const at::Scalar& beta, const at::Scalar& alpha,
                        at::Tensor& out) {
    const c10::DeviceGuard guard(out.device());
    CallContext ctx(out);
    Wrapped o(out), s(self), a(batch1), b(batch2);
    DIPU_B200_CALL(diopiBaddbmm(&ctx, &o, &s, &a, &b, beta.toDouble(), alpha.toDouble()));
    return out;
}

// ---- selection / masks --------------------------------------------------------------------------------------------------------
// yaml:1926-1933; aten::embedding lowers to this (index_select(weight, 0, ids.reshape(-1)) + view)
at::Tensor& index_select_out(const at::Tensor& self, int64_t dim, const at::Tensor& index, at::Tensor& out) {
    const c10::DeviceGuard guard(self.device());
    dim = at::maybe_wrap_dim(dim, self.dim());
    std::vector<int64_t> shape(self.sizes().begin(), self.sizes().end());
    TORCH_CHECK(index.dim() <= 1, "index_select: index must be a vector");
    if (!shape.empty()) shape[dim] = index.numel();
    TORCH_CHECK(out.sizes() == c10::IntArrayRef(shape), "index_select.out: `out` must already have the result shape on dipu");
    CallContext ctx(self);
    Wrapped o(out), s(self), i(index);
    DIPU_B200_CALL(diopiIndexSelect(&ctx, &o, &s, dim, &i));
    return out;
}

at::Tensor index_select(const at::Tensor& self, int64_t dim, const at::Tensor& index) {
    const c10::DeviceGuard guard(self.device());
    std::vector<int64_t> shape(self.sizes().begin(), self.sizes().end());
    if (!shape.empty()) shape[at::maybe_wrap_dim(dim, self.dim())] = index.numel();
    at::Tensor out = at::empty(shape, self.options());
    return index_select_out(self, dim, index, out);
}

// yaml:1418-1430
at::Tensor& cat_out(const at::ITensorListRef& tensors, int64_t dim, at::Tensor& out) {
    const c10::DeviceGuard guard(out.device());
    std::vector<Wrapped> wrapped;
    wrapped.reserve(tensors.size());
    for (const at::Tensor& t : tensors) wrapped.emplace_back(t);
    std::vector<diopiConstTensorHandle_t> handles;
    for (const Wrapped& w : wrapped) handles.push_back(&w);
    CallContext ctx(out);
    Wrapped o(out);
    DIPU_B200_CALL(diopiCat(&ctx, &o, handles.data(), static_cast<int64_t>(handles.size()), at::maybe_wrap_dim(dim, out.dim())));
    return out;
}

// yaml:2507-2516
at::Tensor& triu_out(const at::Tensor& self, int64_t diagonal, at::Tensor& out) {
    const c10::DeviceGuard guard(out.device());
    CallContext ctx(out);
    Wrapped o(out), s(self);
    DIPU_B200_CALL(diopiTriu(&ctx, &o, &s, diagonal));
    return out;
}

// yaml:28-29
at::Tensor& fill_scalar(at::Tensor& self, const at::Scalar& value) {
    const c10::DeviceGuard guard(self.device());
    CallContext ctx(self);
    Wrapped s(self);
    const diopiScalar_t v = to_diopi_scalar(value);
    DIPU_B200_CALL(diopiFill(&ctx, &s, &v));
    return self;
}

at::Tensor& zero_(at::Tensor& self) {
    const c10::DeviceGuard guard(self.device());
    CallContext ctx(self);
    Wrapped s(self);
    DIPU_B200_CALL(diopiZeroInp(&ctx, &s));
    return self;
}

// yaml:1432-1453
at::Tensor& masked_fill_scalar_(at::Tensor& self, const at::Tensor& mask, const at::Scalar& value) {
    const c10::DeviceGuard guard(self.device());
    CallContext ctx(self);
    Wrapped s(self), m(mask);
    const diopiScalar_t v = to_diopi_scalar(value);
    DIPU_B200_CALL(diopiMaskedFillInpScalar(&ctx, &s, &m, &v));
    return self;
}

// yaml:1566-1571
at::Tensor where_self(const at::Tensor& condition, const at::Tensor& self, const at::Tensor& other) {
    const at::Tensor& dev = device_of(device_of(condition, self), other);
    const c10::DeviceGuard guard(dev.device());
    const auto shape = at::infer_size(at::infer_size(condition.sizes(), self.sizes()), other.sizes());
    at::Tensor out = at::empty(shape, dev.options().dtype(at::result_type(self, other)));
    CallContext ctx(out);
    Wrapped o(out), c(condition), s(self), t(other);
    DIPU_B200_CALL(diopiWhere(&ctx, &o, &c, &s, &t));
    return out;
}

// ---- sampling loop (yaml:816-828 topk, 1143-1175 sort, 1516-1519 argmax, 1908-1912 cumsum, 1923-1924 gather, 1199-1211 multinomial)
at::Tensor& argmax_out(const at::Tensor& self, std::optional<int64_t> dim, bool keepdim, at::Tensor& out) {
    const c10::DeviceGuard guard(self.device());
    CallContext ctx(self);
    Wrapped o(out), s(self);
    const int64_t d = dim.has_value() ? *dim : 0;
    DIPU_B200_CALL(diopiArgmax(&ctx, &o, &s, dim.has_value() ? &d : nullptr, keepdim));
    return out;
}

std::tuple<at::Tensor&, at::Tensor&> topk_values(const at::Tensor& self, int64_t k, int64_t dim, bool largest, bool sorted, at::Tensor& values,
                                                 at::Tensor& indices) {
    const c10::DeviceGuard guard(self.device());
    CallContext ctx(self);
    Wrapped v(values), i(indices), s(self);
    DIPU_B200_CALL(diopiTopk(&ctx, &v, &i, &s, k, dim, largest, sorted));
    return {values, indices};
}

std::tuple<at::Tensor&, at::Tensor&> sort_values_stable(const at::Tensor& self, std::optional<bool> stable, int64_t dim, bool descending,
                                                        at::Tensor& values, at::Tensor& indices) {
    const c10::DeviceGuard guard(self.device());
    CallContext ctx(self);
    Wrapped v(values), i(indices), s(self);
    const bool st = stable.value_or(false);
    DIPU_B200_CALL(diopiSort(&ctx, &v, &i, &s, at::maybe_wrap_dim(dim, self.dim()), descending, &st));
    return {values, indices};
}

at::Tensor& cumsum_out(const at::Tensor& self, int64_t dim, std::optional<at::ScalarType> dtype, at::Tensor& out) {
    (void)dtype;  // `out` has the result dtype; the library converts while it loads
    const c10::DeviceGuard guard(self.device());
    CallContext ctx(self);
    Wrapped o(out), s(self);
    DIPU_B200_CALL(diopiCumsum(&ctx, &o, &s, dim));
    return out;
}

at::Tensor& gather_out(const at::Tensor& self, int64_t dim, const at::Tensor& index, bool sparse_grad, at::Tensor& out) {
    (void)sparse_grad;
    const c10::DeviceGuard guard(self.device());
    CallContext ctx(self);
    Wrapped o(out), s(self), i(index);
    DIPU_B200_CALL(diopiGather(&ctx, &o, &s, dim, &i));
    return out;
}

at::Tensor multinomial(const at::Tensor& self, int64_t num_samples, bool replacement, std::optional<at::Generator> generator) {
    TORCH_CHECK(!generator.has_value() || !generator->defined(), "multinomial on dipu: pass no generator (the library's default stream is used)");
    const c10::DeviceGuard guard(self.device());
    at::Tensor out = self.dim() == 2 ? at::empty({self.size(0), num_samples}, self.options().dtype(at::kLong))
                                     : at::empty({num_samples}, self.options().dtype(at::kLong));
    CallContext ctx(self);
    Wrapped o(out), s(self);
    DIPU_B200_CALL(diopiMultinomial(&ctx, &o, &s, num_samples, replacement, nullptr));
    return out;
}

// ---- fused attention: torch.nn.functional.scaled_dot_product_attention ------------------------------------------------------
// torch routes SDPA on a PrivateUse1 device to _scaled_dot_product_fused_attention_overrideable when _fused_sdp_choice
// answers "overrideable" (SDPBackend value 4). q / k / v arrive as [batch, heads, seq, dim] (usually transposed views of the
// projection output); the library takes the [batch, seq, heads, dim] views by their pitches, so nothing is copied.
int64_t fused_sdp_choice(const at::Tensor& query, const at::Tensor& key, const at::Tensor& value, const std::optional<at::Tensor>& attn_mask,
                         double dropout_p, bool is_causal, std::optional<double> scale, bool enable_gqa) {
    (void)key; (void)value; (void)is_causal; (void)scale; (void)enable_gqa;
    const bool fused = !attn_mask.has_value() && dropout_p == 0.0 && query.dim() == 4 && query.size(3) == 128 &&
                       (query.scalar_type() == at::kBFloat16 || query.scalar_type() == at::kHalf);
    return fused ? 4 /* overrideable */ : 0 /* math: the op-by-op composite */;
}

std::tuple<at::Tensor, at::Tensor, at::Tensor, at::Tensor, c10::SymInt, c10::SymInt, at::Tensor, at::Tensor, at::Tensor> sdpa_overrideable(
    const at::Tensor& query, const at::Tensor& key, const at::Tensor& value, const std::optional<at::Tensor>& attn_bias, double dropout_p, bool is_causal,
    bool return_debug_mask, std::optional<double> scale) {
    TORCH_CHECK(!attn_bias.has_value() || !attn_bias->defined(), "fused attention on dipu takes no attn_bias (use is_causal)");
    TORCH_CHECK(query.dim() == 4 && key.dim() == 4 && value.dim() == 4, "fused attention expects [batch, heads, seq, dim] tensors");
    const c10::DeviceGuard guard(query.device());
    const int64_t b = query.size(0), h = query.size(1), sq = query.size(2), d = query.size(3);
    at::Tensor out = at::empty({b, sq, h, d}, query.options());                    // merged layout; returned as its [b, h, sq, d] view
    at::Tensor lse = at::empty({b, h, sq}, query.options().dtype(at::kFloat));
    const at::Tensor q = query.transpose(1, 2), k = key.transpose(1, 2), v = value.transpose(1, 2);
    CallContext ctx(out);
    const double sc = scale.has_value() ? *scale : 1.0 / std::sqrt(static_cast<double>(d));
    auto attend = [&](const at::Tensor& qv, const at::Tensor& kv, const at::Tensor& vv, const at::Tensor& ov, const at::Tensor& lv, bool causal) {
        Wrapped wq(qv), wk(kv), wv(vv), wo(ov), wl(lv);
        DIPU_B200_CALL(diopiMultiHeadAttention(&ctx, &wq, &wk, &wv, dropout_p, causal, return_debug_mask, sc, &wo, &wl, nullptr, nullptr));
    };
    const int64_t skv = key.size(2);
    if (is_causal && sq != skv) {
        // torch aligns the causal mask to the FIRST key (key j is visible to query i iff j <= i, the lower triangle of
        // ones(L, S)); diopiMultiHeadAttention aligns it to the LAST key (j <= i + S - L). The two agree on square problems, so
        // a rectangular one is served as square ones: fewer queries than keys see only the first L keys; with more queries than
        // keys the first S queries form a square causal problem and the remaining ones see every key.
        if (sq < skv) {
            attend(q, k.narrow(1, 0, sq), v.narrow(1, 0, sq), out, lse, true);
        } else {
            attend(q.narrow(1, 0, skv), k, v, out.narrow(1, 0, skv), lse.narrow(2, 0, skv), true);
            attend(q.narrow(1, skv, sq - skv), k, v, out.narrow(1, skv, sq - skv), lse.narrow(2, skv, sq - skv), false);
        }
    } else {
        attend(q, k, v, out, lse, is_causal);
    }
    const at::Tensor none = at::empty({0}, query.options().dtype(at::kLong));
    return {out.transpose(1, 2), lse, none, none, c10::SymInt(sq), c10::SymInt(key.size(2)), none, none, at::empty({0}, query.options())};
}

TORCH_LIBRARY_IMPL(aten, PrivateUse1, m) {
    m.impl("_fused_sdp_choice", &fused_sdp_choice);  // the dispatcher op (Python-visible); SDPA itself asks the stub below
    m.impl("_scaled_dot_product_fused_attention_overrideable", &sdpa_overrideable);
    m.impl("argmax.out", &argmax_out);
    m.impl("topk.values", &topk_values);
    m.impl("sort.values_stable", &sort_values_stable);
    m.impl("cumsum.out", &cumsum_out);
    m.impl("gather.out", &gather_out);
    m.impl("multinomial", &multinomial);
    m.impl("add.out", &add_out);
    m.impl("sub.out", &sub_out);
    m.impl("mul.out", &mul_out);
    m.impl("div.out", &div_out);
    m.impl("silu.out", &silu_out);
    m.impl("neg.out", &neg_out);
    m.impl("rsqrt.out", &rsqrt_out);
    m.impl("sqrt.out", &sqrt_out);
    m.impl("reciprocal.out", &reciprocal_out);
    m.impl("exp.out", &exp_out);
    m.impl("cos.out", &cos_out);
    m.impl("sin.out", &sin_out);
    m.impl("sigmoid.out", &sigmoid_out);
    m.impl("tanh.out", &tanh_out);
    m.impl("pow.Tensor_Scalar_out", &pow_tensor_scalar_out);
    m.impl("mean.out", &mean_out);
    m.impl("_softmax.out", &softmax_out);
    m.impl("native_layer_norm", &native_layer_norm);
    m.impl("_fused_rms_norm", &fused_rms_norm);
    m.impl("mm.out", &mm_out);
    m.impl("bmm.out", &bmm_out);
    m.impl("addmm.out", &addmm_out);
    m.impl("baddbmm.out", &baddbmm_out);
    m.impl("index_select", &index_select);
    m.impl("index_select.out", &index_select_out);
    m.impl("cat.out", &cat_out);
    m.impl("triu.out", &triu_out);
    m.impl("fill_.Scalar", &fill_scalar);
    m.impl("zero_", &zero_);
    m.impl("masked_fill_.Scalar", &masked_fill_scalar_);
    m.impl("where.self", &where_self);
}

}  // namespace
}  // namespace dipu_b200

// scaled_dot_product_attention picks its backend through a dispatch stub, not the dispatcher: the PrivateUse1 slot of that
// stub is this backend's to fill.
namespace at::native {
namespace {
int64_t dipu_b200_sdp_choice(const Tensor& query, const Tensor& key, const Tensor& value, const std::optional<Tensor>& attn_mask, double dropout_p,
                             bool is_causal, std::optional<double> scale, bool enable_gqa) {
    (void)key; (void)value; (void)is_causal; (void)scale; (void)enable_gqa;
    const bool fused = !attn_mask.has_value() && dropout_p == 0.0 && query.dim() == 4 && query.size(3) == 128 &&
                       (query.scalar_type() == at::kBFloat16 || query.scalar_type() == at::kHalf);
    return fused ? 4 /* SDPBackend::overrideable */ : 0 /* SDPBackend::math */;
}
}  // namespace
REGISTER_PRIVATEUSE1_DISPATCH(_fused_sdp_choice_stub, &dipu_b200_sdp_choice)
}  // namespace at::native
