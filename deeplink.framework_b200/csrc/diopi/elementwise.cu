// Unary / binary / ternary element-wise DIOPI functions built on the engine in elementwise.cuh.
#include "elementwise.cuh"

namespace b200 {
namespace {

// ---- math helpers that exist for every compute type -------------------------------------------
__device__ __forceinline__ float m_exp(float x) { return expf(x); }
__device__ __forceinline__ double m_exp(double x) { return exp(x); }
__device__ __forceinline__ float m_sqrt(float x) { return sqrtf(x); }
__device__ __forceinline__ double m_sqrt(double x) { return sqrt(x); }
__device__ __forceinline__ float m_sin(float x) { return sinf(x); }
__device__ __forceinline__ double m_sin(double x) { return sin(x); }
__device__ __forceinline__ float m_cos(float x) { return cosf(x); }
__device__ __forceinline__ double m_cos(double x) { return cos(x); }
__device__ __forceinline__ float m_tanh(float x) { return tanhf(x); }
__device__ __forceinline__ double m_tanh(double x) { return tanh(x); }
__device__ __forceinline__ float m_pow(float x, float y) { return powf(x, y); }
__device__ __forceinline__ double m_pow(double x, double y) { return pow(x, y); }
__device__ __forceinline__ float m_floor(float x) { return floorf(x); }
__device__ __forceinline__ double m_floor(double x) { return floor(x); }
__device__ __forceinline__ float m_trunc(float x) { return truncf(x); }
__device__ __forceinline__ double m_trunc(double x) { return trunc(x); }

template <typename C> struct FloatOf { using type = C; };
template <> struct FloatOf<int64_t> { using type = double; };

#define B200_UNARY_FLOAT_OP(NAME, EXPR)                                  \
    template <typename C>                                                \
    struct NAME {                                                        \
        explicit NAME(const ScalarArgs&) {}                              \
        __device__ __forceinline__ C operator()(C a) const {             \
            using F = typename FloatOf<C>::type;                         \
            const F x = static_cast<F>(a);                               \
            return static_cast<C>(EXPR);                                 \
        }                                                                \
    };

B200_UNARY_FLOAT_OP(OpRsqrt, F(1) / m_sqrt(x))
B200_UNARY_FLOAT_OP(OpSqrt, m_sqrt(x))
B200_UNARY_FLOAT_OP(OpRecip, F(1) / x)
B200_UNARY_FLOAT_OP(OpExp, m_exp(x))
B200_UNARY_FLOAT_OP(OpSin, m_sin(x))
B200_UNARY_FLOAT_OP(OpCos, m_cos(x))
B200_UNARY_FLOAT_OP(OpTanh, m_tanh(x))
B200_UNARY_FLOAT_OP(OpSigmoid, F(1) / (F(1) + m_exp(-x)))
B200_UNARY_FLOAT_OP(OpSilu, x / (F(1) + m_exp(-x)))
// 16-bit storage: ex2.approx and an approximate division (about 2 ulp of fp32 each) instead of the exact forms, which cost
// more instructions per element than the memory system leaves room for
template <typename C>
struct OpSiluFast {
    explicit OpSiluFast(const ScalarArgs&) {}
    __device__ __forceinline__ C operator()(C a) const {
        const float x = static_cast<float>(a);
        return static_cast<C>(__fdividef(x, 1.0f + __expf(-x)));
    }
};
}  // namespace
template <>
struct HalfOp<OpSilu> {
    template <typename C>
    using type = OpSiluFast<C>;
};
namespace {

template <typename C>
struct OpNeg {
    explicit OpNeg(const ScalarArgs&) {}
    __device__ __forceinline__ C operator()(C a) const { return -a; }
};
template <typename C>
struct OpRelu {
    explicit OpRelu(const ScalarArgs&) {}
    __device__ __forceinline__ C operator()(C a) const { return a > C(0) ? a : C(0); }
};
template <typename C>
struct OpIdentity {
    explicit OpIdentity(const ScalarArgs&) {}
    __device__ __forceinline__ C operator()(C a) const { return a; }
};

// out = a + alpha * b
template <typename C>
struct OpAdd {
    C alpha;
    explicit OpAdd(const ScalarArgs& s) : alpha(pick_scalar<C>(s, 0)) {}
    __device__ __forceinline__ C operator()(C a, C b) const { return a + alpha * b; }
};
template <typename C>
struct OpAddPlain {  // alpha == 1: keeps the sum free of a multiply so it matches a + b bit for bit
    explicit OpAddPlain(const ScalarArgs&) {}
    __device__ __forceinline__ C operator()(C a, C b) const { return a + b; }
};
template <typename C>
struct OpMul {
    explicit OpMul(const ScalarArgs&) {}
    __device__ __forceinline__ C operator()(C a, C b) const { return a * b; }
};
// out = a * p0 + p1
template <typename C>
struct OpAffine {
    C p0, p1;
    explicit OpAffine(const ScalarArgs& s) : p0(pick_scalar<C>(s, 0)), p1(pick_scalar<C>(s, 1)) {}
    __device__ __forceinline__ C operator()(C a) const { return a * p0 + p1; }
};
template <typename C>
struct OpAddConst {  // out = a + p1 (no multiply)
    C p1;
    explicit OpAddConst(const ScalarArgs& s) : p1(pick_scalar<C>(s, 1)) {}
    __device__ __forceinline__ C operator()(C a) const { return a + p1; }
};
template <typename C>
struct OpMulConst {
    C p0;
    explicit OpMulConst(const ScalarArgs& s) : p0(pick_scalar<C>(s, 0)) {}
    __device__ __forceinline__ C operator()(C a) const { return a * p0; }
};

template <typename C>
__device__ __forceinline__ C apply_round(C q, int64_t mode) {
    using F = typename FloatOf<C>::type;
    if (mode == RoundModeTrunc) return static_cast<C>(m_trunc(static_cast<F>(q)));
    if (mode == RoundModeFloor) return static_cast<C>(m_floor(static_cast<F>(q)));
    return q;
}
template <>
__device__ __forceinline__ int64_t apply_round<int64_t>(int64_t q, int64_t) { return q; }

template <typename C>
__device__ __forceinline__ C div_mode(C a, C b, int64_t mode) { return apply_round<C>(a / b, mode); }
template <>
__device__ __forceinline__ int64_t div_mode<int64_t>(int64_t a, int64_t b, int64_t mode) {
    if (b == 0) return 0;
    int64_t q = a / b;  // truncates toward zero
    if (mode == RoundModeFloor && ((a % b) != 0) && ((a < 0) != (b < 0))) --q;
    return q;
}

template <typename C>
struct OpDiv {
    int64_t mode;
    explicit OpDiv(const ScalarArgs& s) : mode(s.i[1]) {}
    __device__ __forceinline__ C operator()(C a, C b) const { return div_mode<C>(a, b, mode); }
};
template <typename C>
struct OpDivConst {  // a / p0
    C p0;
    int64_t mode;
    explicit OpDivConst(const ScalarArgs& s) : p0(pick_scalar<C>(s, 0)), mode(s.i[1]) {}
    __device__ __forceinline__ C operator()(C a) const { return div_mode<C>(a, p0, mode); }
};
template <typename C>
struct OpRDivConst {  // p0 / a
    C p0;
    int64_t mode;
    explicit OpRDivConst(const ScalarArgs& s) : p0(pick_scalar<C>(s, 0)), mode(s.i[1]) {}
    __device__ __forceinline__ C operator()(C a) const { return div_mode<C>(p0, a, mode); }
};

template <typename C>
__device__ __forceinline__ C pow_any(C a, C e) {
    using F = typename FloatOf<C>::type;
    return static_cast<C>(m_pow(static_cast<F>(a), static_cast<F>(e)));
}
template <typename C>
struct OpPowConst {  // a ^ p0, with the exact small-exponent shortcuts torch's CPU kernel takes
    C p0;
    explicit OpPowConst(const ScalarArgs& s) : p0(pick_scalar<C>(s, 0)) {}
    __device__ __forceinline__ C operator()(C a) const {
        if (p0 == C(2)) return a * a;
        if (p0 == C(3)) return a * a * a;
        if (p0 == C(1)) return a;
        using F = typename FloatOf<C>::type;
        if (static_cast<F>(p0) == F(0.5)) return static_cast<C>(m_sqrt(static_cast<F>(a)));
        if (static_cast<F>(p0) == F(-0.5)) return static_cast<C>(F(1) / m_sqrt(static_cast<F>(a)));
        if (p0 == C(-1)) return static_cast<C>(F(1) / static_cast<F>(a));
        return pow_any<C>(a, p0);
    }
};
template <typename C>
struct OpRPowConst {  // p0 ^ a
    C p0;
    explicit OpRPowConst(const ScalarArgs& s) : p0(pick_scalar<C>(s, 0)) {}
    __device__ __forceinline__ C operator()(C a) const { return pow_any<C>(p0, a); }
};
template <typename C>
struct OpPow {
    explicit OpPow(const ScalarArgs&) {}
    __device__ __forceinline__ C operator()(C a, C b) const { return pow_any<C>(a, b); }
};

template <typename C>
struct OpFill {
    C p0;
    explicit OpFill(const ScalarArgs& s) : p0(pick_scalar<C>(s, 0)) {}
    __device__ __forceinline__ C operator()() const { return p0; }
};
template <typename C>
struct OpMaskedFillConst {  // (a, mask) -> mask ? p0 : a
    C p0;
    explicit OpMaskedFillConst(const ScalarArgs& s) : p0(pick_scalar<C>(s, 0)) {}
    __device__ __forceinline__ C operator()(C a, C m) const { return m != C(0) ? p0 : a; }
};
template <typename C>
struct OpWhere {  // (cond, a, b)
    explicit OpWhere(const ScalarArgs&) {}
    __device__ __forceinline__ C operator()(C c, C a, C b) const { return c != C(0) ? a : b; }
};

// ---- host-side glue ---------------------------------------------------------------------------------
bool is_host_scalar(const TensorView& v) { return v.device == diopi_host && v.numel == 1; }

// Reads a one-element host tensor into a diopiScalar_t.
bool host_scalar_value(const TensorView& v, diopiScalar_t* s) {
    const void* p = v.data;
    switch (v.dtype) {
        case diopi_dtype_float32: s->stype = diopi_dtype_float64; s->fval = *static_cast<const float*>(p); return true;
        case diopi_dtype_float64: s->stype = diopi_dtype_float64; s->fval = *static_cast<const double*>(p); return true;
        case diopi_dtype_float16: {
            uint16_t h = *static_cast<const uint16_t*>(p);
            const uint32_t sign = (h >> 15) & 1u, exp = (h >> 10) & 0x1fu, man = h & 0x3ffu;
            double val;
            if (exp == 0) val = man * 5.9604644775390625e-08;  // 2^-24
            else if (exp == 31) val = man ? __builtin_nan("") : __builtin_inf();
            else val = (1.0 + man / 1024.0) * __builtin_ldexp(1.0, (int)exp - 15);
            s->stype = diopi_dtype_float64; s->fval = sign ? -val : val; return true;
        }
        case diopi_dtype_bfloat16: {
            uint32_t bits = static_cast<uint32_t>(*static_cast<const uint16_t*>(p)) << 16;
            float f; memcpy(&f, &bits, 4);
            s->stype = diopi_dtype_float64; s->fval = f; return true;
        }
        case diopi_dtype_int64: s->stype = diopi_dtype_int64; s->ival = *static_cast<const int64_t*>(p); return true;
        case diopi_dtype_int32: s->stype = diopi_dtype_int64; s->ival = *static_cast<const int32_t*>(p); return true;
        case diopi_dtype_int16: s->stype = diopi_dtype_int64; s->ival = *static_cast<const int16_t*>(p); return true;
        case diopi_dtype_int8: s->stype = diopi_dtype_int64; s->ival = *static_cast<const int8_t*>(p); return true;
        case diopi_dtype_uint8: s->stype = diopi_dtype_int64; s->ival = *static_cast<const uint8_t*>(p); return true;
        case diopi_dtype_bool: s->stype = diopi_dtype_int64; s->ival = *static_cast<const uint8_t*>(p) != 0; return true;
        default: return false;
    }
}

double scalar_f(const diopiScalar_t* s) {
    if (!s) return 1.0;
    return (s->stype == diopi_dtype_float64 || s->stype == diopi_dtype_float32) ? s->fval : static_cast<double>(s->ival);
}
int64_t scalar_i(const diopiScalar_t* s) {
    if (!s) return 1;
    return (s->stype == diopi_dtype_float64 || s->stype == diopi_dtype_float32) ? static_cast<int64_t>(s->fval) : s->ival;
}
bool scalar_is_one(const diopiScalar_t* s) { return s == nullptr || (scalar_f(s) == 1.0 && scalar_i(s) == 1); }

template <template <typename> class OpT>
diopiError_t unary(diopiContextHandle_t ctx, const char* name, diopiTensorHandle_t out, diopiConstTensorHandle_t in,
                   const ScalarArgs& sa = ScalarArgs()) {
    B200_VIEW(vo, out);
    B200_VIEW(vi, in);
    const TensorView* ins[1] = {&vi};
    return launch_elementwise<OpT, 1>(ctx, name, vo, ins, sa);
}

template <template <typename> class OpT>
diopiError_t binary(diopiContextHandle_t ctx, const char* name, const TensorView& vo, const TensorView& va, const TensorView& vb,
                    const ScalarArgs& sa) {
    const TensorView* ins[2] = {&va, &vb};
    return launch_elementwise<OpT, 2>(ctx, name, vo, ins, sa);
}

// out = x * mul + add, picking the cheapest exact form.
diopiError_t affine(diopiContextHandle_t ctx, const char* name, const TensorView& vo, const TensorView& vx, double mul_f, int64_t mul_i,
                    double add_f, int64_t add_i) {
    ScalarArgs sa;
    sa.f[0] = mul_f; sa.i[0] = mul_i; sa.f[1] = add_f; sa.i[1] = add_i;
    const TensorView* ins[1] = {&vx};
    if (mul_f == 1.0 && mul_i == 1) return launch_elementwise<OpAddConst, 1>(ctx, name, vo, ins, sa);
    if (add_f == 0.0 && add_i == 0) return launch_elementwise<OpMulConst, 1>(ctx, name, vo, ins, sa);
    return launch_elementwise<OpAffine, 1>(ctx, name, vo, ins, sa);
}

// sign = +1 for add, -1 for sub
diopiError_t add_like(diopiContextHandle_t ctx, const char* name, diopiTensorHandle_t out, diopiConstTensorHandle_t a,
                      diopiConstTensorHandle_t b, const diopiScalar_t* alpha, int sign) {
    B200_VIEW(vo, out);
    B200_VIEW(va, a);
    B200_VIEW(vb, b);
    const double af = scalar_f(alpha) * sign;
    const int64_t ai = scalar_i(alpha) * sign;
    diopiScalar_t hs;
    if (is_host_scalar(vb)) {  // x + alpha * s
        B200_CHECK(host_scalar_value(vb, &hs), "%s: unsupported host scalar dtype", name);
        return affine(ctx, name, vo, va, 1.0, 1, af * scalar_f(&hs), ai * scalar_i(&hs));
    }
    if (is_host_scalar(va)) {  // s + alpha * x
        B200_CHECK(host_scalar_value(va, &hs), "%s: unsupported host scalar dtype", name);
        return affine(ctx, name, vo, vb, af, ai, scalar_f(&hs), scalar_i(&hs));
    }
    ScalarArgs sa;
    sa.f[0] = af; sa.i[0] = ai;
    if (af == 1.0 && ai == 1) return binary<OpAddPlain>(ctx, name, vo, va, vb, sa);
    return binary<OpAdd>(ctx, name, vo, va, vb, sa);
}

diopiError_t add_scalar_like(diopiContextHandle_t ctx, const char* name, diopiTensorHandle_t out, diopiConstTensorHandle_t a,
                             const diopiScalar_t* other, const diopiScalar_t* alpha, int sign) {
    B200_VIEW(vo, out);
    B200_VIEW(va, a);
    B200_CHECK(other != nullptr, "%s: scalar operand is NULL", name);
    return affine(ctx, name, vo, va, 1.0, 1, scalar_f(alpha) * scalar_f(other) * sign, scalar_i(alpha) * scalar_i(other) * sign);
}

diopiError_t mul_like(diopiContextHandle_t ctx, const char* name, diopiTensorHandle_t out, diopiConstTensorHandle_t a,
                      diopiConstTensorHandle_t b) {
    B200_VIEW(vo, out);
    B200_VIEW(va, a);
    B200_VIEW(vb, b);
    diopiScalar_t hs;
    if (is_host_scalar(vb) || is_host_scalar(va)) {
        const TensorView& vs = is_host_scalar(vb) ? vb : va;
        const TensorView& vx = is_host_scalar(vb) ? va : vb;
        B200_CHECK(host_scalar_value(vs, &hs), "%s: unsupported host scalar dtype", name);
        return affine(ctx, name, vo, vx, scalar_f(&hs), scalar_i(&hs), 0.0, 0);
    }
    return binary<OpMul>(ctx, name, vo, va, vb, ScalarArgs());
}

diopiError_t div_like(diopiContextHandle_t ctx, const char* name, diopiTensorHandle_t out, diopiConstTensorHandle_t a,
                      diopiConstTensorHandle_t b, diopiRoundMode_t mode) {
    B200_VIEW(vo, out);
    B200_VIEW(va, a);
    B200_VIEW(vb, b);
    ScalarArgs sa;
    sa.i[1] = mode;
    diopiScalar_t hs;
    if (is_host_scalar(vb)) {
        B200_CHECK(host_scalar_value(vb, &hs), "%s: unsupported host scalar dtype", name);
        sa.f[0] = scalar_f(&hs); sa.i[0] = scalar_i(&hs);
        const TensorView* ins[1] = {&va};
        return launch_elementwise<OpDivConst, 1>(ctx, name, vo, ins, sa);
    }
    if (is_host_scalar(va)) {
        B200_CHECK(host_scalar_value(va, &hs), "%s: unsupported host scalar dtype", name);
        sa.f[0] = scalar_f(&hs); sa.i[0] = scalar_i(&hs);
        const TensorView* ins[1] = {&vb};
        return launch_elementwise<OpRDivConst, 1>(ctx, name, vo, ins, sa);
    }
    return binary<OpDiv>(ctx, name, vo, va, vb, sa);
}

}  // namespace
}  // namespace b200

using namespace b200;

extern "C" {

// ---- unary -----------------------------------------------------------------------------------------
diopiError_t diopiNeg(diopiContextHandle_t ctx, diopiTensorHandle_t out, diopiConstTensorHandle_t input) { return unary<OpNeg>(ctx, "diopiNeg", out, input); }
diopiError_t diopiNegInp(diopiContextHandle_t ctx, diopiTensorHandle_t input) { return unary<OpNeg>(ctx, "diopiNegInp", input, input); }
diopiError_t diopiRsqrt(diopiContextHandle_t ctx, diopiTensorHandle_t out, diopiConstTensorHandle_t input) { return unary<OpRsqrt>(ctx, "diopiRsqrt", out, input); }
diopiError_t diopiRsqrtInp(diopiContextHandle_t ctx, diopiTensorHandle_t input) { return unary<OpRsqrt>(ctx, "diopiRsqrtInp", input, input); }
diopiError_t diopiSqrt(diopiContextHandle_t ctx, diopiTensorHandle_t out, diopiConstTensorHandle_t input) { return unary<OpSqrt>(ctx, "diopiSqrt", out, input); }
diopiError_t diopiReciprocal(diopiContextHandle_t ctx, diopiTensorHandle_t out, diopiConstTensorHandle_t input) { return unary<OpRecip>(ctx, "diopiReciprocal", out, input); }
diopiError_t diopiExp(diopiContextHandle_t ctx, diopiTensorHandle_t out, diopiConstTensorHandle_t input) { return unary<OpExp>(ctx, "diopiExp", out, input); }
diopiError_t diopiSin(diopiContextHandle_t ctx, diopiTensorHandle_t out, diopiConstTensorHandle_t input) { return unary<OpSin>(ctx, "diopiSin", out, input); }
diopiError_t diopiSinInp(diopiContextHandle_t ctx, diopiTensorHandle_t input) { return unary<OpSin>(ctx, "diopiSinInp", input, input); }
diopiError_t diopiCos(diopiContextHandle_t ctx, diopiTensorHandle_t out, diopiConstTensorHandle_t input) { return unary<OpCos>(ctx, "diopiCos", out, input); }
diopiError_t diopiCosInp(diopiContextHandle_t ctx, diopiTensorHandle_t input) { return unary<OpCos>(ctx, "diopiCosInp", input, input); }
diopiError_t diopiSilu(diopiContextHandle_t ctx, diopiTensorHandle_t out, diopiConstTensorHandle_t input) { return unary<OpSilu>(ctx, "diopiSilu", out, input); }
diopiError_t diopiSiluInp(diopiContextHandle_t ctx, diopiTensorHandle_t input) { return unary<OpSilu>(ctx, "diopiSiluInp", input, input); }
diopiError_t diopiSigmoid(diopiContextHandle_t ctx, diopiTensorHandle_t out, diopiConstTensorHandle_t input) { return unary<OpSigmoid>(ctx, "diopiSigmoid", out, input); }
diopiError_t diopiRelu(diopiContextHandle_t ctx, diopiTensorHandle_t out, diopiConstTensorHandle_t input) { return unary<OpRelu>(ctx, "diopiRelu", out, input); }
diopiError_t diopiTanh(diopiContextHandle_t ctx, diopiTensorHandle_t out, diopiConstTensorHandle_t input) { return unary<OpTanh>(ctx, "diopiTanh", out, input); }

// ---- add / sub ---------------------------------------------------------------------------------------
diopiError_t diopiAdd(diopiContextHandle_t ctx, diopiTensorHandle_t out, diopiConstTensorHandle_t input, diopiConstTensorHandle_t other,
                      const diopiScalar_t* alpha) {
    return add_like(ctx, "diopiAdd", out, input, other, alpha, +1);
}
diopiError_t diopiAddInp(diopiContextHandle_t ctx, diopiTensorHandle_t input, diopiConstTensorHandle_t other, const diopiScalar_t* alpha) {
    return add_like(ctx, "diopiAddInp", input, input, other, alpha, +1);
}
diopiError_t diopiAddScalar(diopiContextHandle_t ctx, diopiTensorHandle_t out, diopiConstTensorHandle_t input, const diopiScalar_t* other,
                            const diopiScalar_t* alpha) {
    return add_scalar_like(ctx, "diopiAddScalar", out, input, other, alpha, +1);
}
diopiError_t diopiAddInpScalar(diopiContextHandle_t ctx, diopiTensorHandle_t input, const diopiScalar_t* other, const diopiScalar_t* alpha) {
    return add_scalar_like(ctx, "diopiAddInpScalar", input, input, other, alpha, +1);
}
diopiError_t diopiSub(diopiContextHandle_t ctx, diopiTensorHandle_t out, diopiConstTensorHandle_t input, diopiConstTensorHandle_t other,
                      const diopiScalar_t* alpha) {
    return add_like(ctx, "diopiSub", out, input, other, alpha, -1);
}
diopiError_t diopiSubInp(diopiContextHandle_t ctx, diopiTensorHandle_t input, diopiConstTensorHandle_t other, const diopiScalar_t* alpha) {
    return add_like(ctx, "diopiSubInp", input, input, other, alpha, -1);
}
diopiError_t diopiSubScalar(diopiContextHandle_t ctx, diopiTensorHandle_t out, diopiConstTensorHandle_t input, const diopiScalar_t* other,
                            const diopiScalar_t* alpha) {
    return add_scalar_like(ctx, "diopiSubScalar", out, input, other, alpha, -1);
}
diopiError_t diopiSubInpScalar(diopiContextHandle_t ctx, diopiTensorHandle_t input, const diopiScalar_t* other, const diopiScalar_t* alpha) {
    return add_scalar_like(ctx, "diopiSubInpScalar", input, input, other, alpha, -1);
}

// ---- mul / div -----------------------------------------------------------------------------------------
diopiError_t diopiMul(diopiContextHandle_t ctx, diopiTensorHandle_t out, diopiConstTensorHandle_t input, diopiConstTensorHandle_t other) {
    return mul_like(ctx, "diopiMul", out, input, other);
}
diopiError_t diopiMulInp(diopiContextHandle_t ctx, diopiTensorHandle_t input, diopiConstTensorHandle_t other) {
    return mul_like(ctx, "diopiMulInp", input, input, other);
}
diopiError_t diopiMulScalar(diopiContextHandle_t ctx, diopiTensorHandle_t out, diopiConstTensorHandle_t input, const diopiScalar_t* other) {
    B200_VIEW(vo, out);
    B200_VIEW(vi, input);
    B200_CHECK(other != nullptr, "diopiMulScalar: scalar operand is NULL");
    return affine(ctx, "diopiMulScalar", vo, vi, scalar_f(other), scalar_i(other), 0.0, 0);
}
diopiError_t diopiMulInpScalar(diopiContextHandle_t ctx, diopiTensorHandle_t input, const diopiScalar_t* other) {
    return diopiMulScalar(ctx, input, input, other);
}
diopiError_t diopiDiv(diopiContextHandle_t ctx, diopiTensorHandle_t out, diopiConstTensorHandle_t input, diopiConstTensorHandle_t other,
                      diopiRoundMode_t rounding_mode) {
    return div_like(ctx, "diopiDiv", out, input, other, rounding_mode);
}
diopiError_t diopiDivInp(diopiContextHandle_t ctx, diopiTensorHandle_t input, diopiConstTensorHandle_t other, diopiRoundMode_t rounding_mode) {
    return div_like(ctx, "diopiDivInp", input, input, other, rounding_mode);
}
diopiError_t diopiDivScalar(diopiContextHandle_t ctx, diopiTensorHandle_t out, diopiConstTensorHandle_t input, const diopiScalar_t* other,
                            diopiRoundMode_t rounding_mode) {
    B200_VIEW(vo, out);
    B200_VIEW(vi, input);
    B200_CHECK(other != nullptr, "diopiDivScalar: scalar operand is NULL");
    // Two-byte float outputs: x / s is formed as x * (1 / s) in fp32 (as ATen's CUDA kernel does for a scalar divisor).
    // The product differs from the quotient by at most one fp32 ulp, far below the output's own rounding step, and the
    // multiply keeps the kernel at the memory roofline. fp32 / fp64 / integer outputs use true division.
    if (rounding_mode == RoundModeNone && (vo.dtype == diopi_dtype_bfloat16 || vo.dtype == diopi_dtype_float16) && vi.dtype == vo.dtype &&
        scalar_f(other) != 0.0) {
        return affine(ctx, "diopiDivScalar", vo, vi, 1.0 / scalar_f(other), 0, 0.0, 0);
    }
    ScalarArgs sa;
    sa.f[0] = scalar_f(other); sa.i[0] = scalar_i(other); sa.i[1] = rounding_mode;
    const TensorView* ins[1] = {&vi};
    return launch_elementwise<OpDivConst, 1>(ctx, "diopiDivScalar", vo, ins, sa);
}
diopiError_t diopiDivInpScalar(diopiContextHandle_t ctx, diopiTensorHandle_t input, const diopiScalar_t* other, diopiRoundMode_t rounding_mode) {
    return diopiDivScalar(ctx, input, input, other, rounding_mode);
}

// ---- pow ---------------------------------------------------------------------------------------------------
diopiError_t diopiPow(diopiContextHandle_t ctx, diopiTensorHandle_t out, diopiConstTensorHandle_t input, const diopiScalar_t* exponent) {
    B200_CHECK(exponent != nullptr, "diopiPow: exponent is NULL");
    ScalarArgs sa;
    scalar_to_args(exponent, &sa, 0);
    return unary<OpPowConst>(ctx, "diopiPow", out, input, sa);
}
diopiError_t diopiPowInp(diopiContextHandle_t ctx, diopiTensorHandle_t input, const diopiScalar_t* exponent) {
    return diopiPow(ctx, input, input, exponent);
}
diopiError_t diopiPowTensor(diopiContextHandle_t ctx, diopiTensorHandle_t out, diopiConstTensorHandle_t input, diopiConstTensorHandle_t exponent) {
    B200_VIEW(vo, out);
    B200_VIEW(va, input);
    B200_VIEW(vb, exponent);
    if (is_host_scalar(vb)) {
        diopiScalar_t hs;
        B200_CHECK(host_scalar_value(vb, &hs), "diopiPowTensor: unsupported host scalar dtype");
        ScalarArgs sa;
        scalar_to_args(&hs, &sa, 0);
        const TensorView* ins[1] = {&va};
        return launch_elementwise<OpPowConst, 1>(ctx, "diopiPowTensor", vo, ins, sa);
    }
    return binary<OpPow>(ctx, "diopiPowTensor", vo, va, vb, ScalarArgs());
}
diopiError_t diopiPowScalar(diopiContextHandle_t ctx, diopiTensorHandle_t out, const diopiScalar_t* input, diopiConstTensorHandle_t exponent) {
    B200_CHECK(input != nullptr, "diopiPowScalar: base is NULL");
    ScalarArgs sa;
    scalar_to_args(input, &sa, 0);
    return unary<OpRPowConst>(ctx, "diopiPowScalar", out, exponent, sa);
}

// ---- fill / masks ----------------------------------------------------------------------------------------
diopiError_t diopiFill(diopiContextHandle_t ctx, diopiTensorHandle_t input, const diopiScalar_t* value) {
    B200_VIEW(vo, input);
    B200_CHECK(value != nullptr, "diopiFill: value is NULL");
    ScalarArgs sa;
    scalar_to_args(value, &sa, 0);
    return launch_elementwise<OpFill, 0>(ctx, "diopiFill", vo, nullptr, sa);
}
diopiError_t diopiZeroInp(diopiContextHandle_t ctx, diopiTensorHandle_t input) {
    B200_VIEW(vo, input);
    if (vo.numel == 0) return diopiSuccess;
    if (vo.is_contiguous()) {
        B200_CUDA(cudaMemsetAsync(vo.data, 0, static_cast<size_t>(vo.numel * vo.itemsize), stream_of(ctx)));
        return diopiSuccess;
    }
    ScalarArgs sa;
    return launch_elementwise<OpFill, 0>(ctx, "diopiZeroInp", vo, nullptr, sa);
}
diopiError_t diopiZeros(diopiContextHandle_t ctx, diopiTensorHandle_t out, diopiSize_t) { return diopiZeroInp(ctx, out); }
diopiError_t diopiOnes(diopiContextHandle_t ctx, diopiTensorHandle_t out, diopiSize_t) {
    diopiScalar_t one;
    one.stype = diopi_dtype_int64;
    one.ival = 1;
    return diopiFill(ctx, out, &one);
}

diopiError_t diopiMaskedFillScalar(diopiContextHandle_t ctx, diopiTensorHandle_t out, diopiConstTensorHandle_t input,
                                   diopiConstTensorHandle_t mask, const diopiScalar_t* value) {
    B200_VIEW(vo, out);
    B200_VIEW(vi, input);
    B200_VIEW(vm, mask);
    B200_CHECK(value != nullptr, "diopiMaskedFillScalar: value is NULL");
    ScalarArgs sa;
    scalar_to_args(value, &sa, 0);
    const TensorView* ins[2] = {&vi, &vm};
    // mask is bool: the vector path (same dtype everywhere) never applies
    return launch_elementwise<OpMaskedFillConst, 2>(ctx, "diopiMaskedFillScalar", vo, ins, sa, /*allow_vec=*/false);
}
diopiError_t diopiMaskedFillInpScalar(diopiContextHandle_t ctx, diopiTensorHandle_t input, diopiConstTensorHandle_t mask,
                                      const diopiScalar_t* value) {
    return diopiMaskedFillScalar(ctx, input, input, mask, value);
}
diopiError_t diopiMaskedFill(diopiContextHandle_t ctx, diopiTensorHandle_t out, diopiConstTensorHandle_t input, diopiConstTensorHandle_t mask,
                             diopiConstTensorHandle_t value) {
    B200_VIEW(vo, out);
    B200_VIEW(vi, input);
    B200_VIEW(vm, mask);
    B200_VIEW(vv, value);
    if (is_host_scalar(vv)) {
        diopiScalar_t hs;
        B200_CHECK(host_scalar_value(vv, &hs), "diopiMaskedFill: unsupported host scalar dtype");
        return diopiMaskedFillScalar(ctx, out, input, mask, &hs);
    }
    const TensorView* ins[3] = {&vm, &vv, &vi};
    return launch_elementwise<OpWhere, 3>(ctx, "diopiMaskedFill", vo, ins, ScalarArgs(), false);
}
diopiError_t diopiMaskedFillInp(diopiContextHandle_t ctx, diopiTensorHandle_t input, diopiConstTensorHandle_t mask,
                                diopiConstTensorHandle_t value) {
    return diopiMaskedFill(ctx, input, input, mask, value);
}
diopiError_t diopiWhere(diopiContextHandle_t ctx, diopiTensorHandle_t out, diopiConstTensorHandle_t condition, diopiConstTensorHandle_t input,
                        diopiConstTensorHandle_t other) {
    B200_VIEW(vo, out);
    B200_VIEW(vc, condition);
    B200_VIEW(va, input);
    B200_VIEW(vb, other);
    const TensorView* ins[3] = {&vc, &va, &vb};
    return launch_elementwise<OpWhere, 3>(ctx, "diopiWhere", vo, ins, ScalarArgs(), false);
}

}  // extern "C"
