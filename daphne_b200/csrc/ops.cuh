// Scalar semantics of the elementwise op codes, written so that the device result has the bits of the
// reference's CPU scalar kernels (src/runtime/local/kernels/EwBinarySca.h:138-166, EwUnarySca.h:182-206):
// every arithmetic step is a single correctly rounded IEEE operation issued through the *_rn intrinsics, which the
// compiler never contracts into FMAs; MIN/MAX are std::min/std::max (so NaN and signed-zero cases pick the same
// operand as on the CPU); comparisons and logical ops yield 0/1 in the value type.
#pragma once

#include "common.cuh"

namespace db2 {

template <typename VT> __device__ __forceinline__ VT op_add(VT a, VT b) {
    if constexpr (std::is_same_v<VT, double>)
        return __dadd_rn(a, b);
    else if constexpr (std::is_same_v<VT, float>)
        return __fadd_rn(a, b);
    else
        return (VT)((uint64_t)a + (uint64_t)b);
}
template <typename VT> __device__ __forceinline__ VT op_sub(VT a, VT b) {
    if constexpr (std::is_same_v<VT, double>)
        return __dsub_rn(a, b);
    else if constexpr (std::is_same_v<VT, float>)
        return __fsub_rn(a, b);
    else
        return (VT)((uint64_t)a - (uint64_t)b);
}
template <typename VT> __device__ __forceinline__ VT op_mul(VT a, VT b) {
    if constexpr (std::is_same_v<VT, double>)
        return __dmul_rn(a, b);
    else if constexpr (std::is_same_v<VT, float>)
        return __fmul_rn(a, b);
    else
        return (VT)((uint64_t)a * (uint64_t)b);
}
template <typename VT> __device__ __forceinline__ VT op_div(VT a, VT b) {
    if constexpr (std::is_same_v<VT, double>)
        return __ddiv_rn(a, b);
    else if constexpr (std::is_same_v<VT, float>)
        return __fdiv_rn(a, b);
    else {
        // integer division by zero terminates the reference process (SIGFPE); here it yields 0
        if (b == 0)
            return 0;
        if constexpr (std::is_signed_v<VT>) { // the one quotient that does not fit the type
            if (a == std::numeric_limits<VT>::min() && b == (VT)-1)
                return std::numeric_limits<VT>::min();
        }
        return a / b;
    }
}
// pow: the exponents 2, 1, 0.5 are evaluated with one correctly rounded operation; everything else goes through
// CUDA's pow (documented maximum error 2 ulp for double).
template <typename VT> __device__ __forceinline__ VT op_pow(VT a, VT b) {
    if constexpr (std::is_same_v<VT, double>) {
        if (b == 2.0)
            return __dmul_rn(a, a);
        if (b == 1.0)
            return a;
        return pow(a, b);
    } else if constexpr (std::is_same_v<VT, float>) {
        // the reference promotes float arguments of pow() to double (unqualified ::pow)
        return (float)pow((double)a, (double)b);
    } else {
        // integer value types: the reference evaluates pow(double(a), double(b)) with glibc, which returns the exact
        // power whenever it is representable, and truncates.  A power with a small non-negative integer exponent is
        // therefore formed by exact multiplications (every partial product below 2^53 is exact); CUDA's pow may be an
        // ulp low and would truncate to the integer below.
        const double x = (double)a, y = (double)b;
        if (y >= 0.0 && y <= 64.0) {
            double r = 1.0, p = x;
            for (unsigned e = (unsigned)y; e; e >>= 1) {
                if (e & 1u)
                    r = __dmul_rn(r, p);
                p = __dmul_rn(p, p);
            }
            return (VT)r;
        }
        return (VT)pow(x, y);
    }
}
template <typename VT> __device__ __forceinline__ VT op_mod(VT a, VT b) {
    if constexpr (std::is_same_v<VT, double>)
        return fmod(a, b);
    else if constexpr (std::is_same_v<VT, float>)
        return fmodf(a, b);
    else
        return (VT)fmod((double)a, (double)b);
}
template <typename VT> __device__ __forceinline__ VT op_log(VT a, VT b) {
    if constexpr (std::is_same_v<VT, float>)
        return __fdiv_rn(logf(a), logf(b));
    else if constexpr (std::is_same_v<VT, double>)
        return __ddiv_rn(log(a), log(b));
    else
        return (VT)__ddiv_rn(log((double)a), log((double)b));
}
template <typename VT> __device__ __forceinline__ VT op_min(VT a, VT b) { return (b < a) ? b : a; }
template <typename VT> __device__ __forceinline__ VT op_max(VT a, VT b) { return (a < b) ? b : a; }

template <int OP, typename VT> __device__ __forceinline__ VT binary_op(VT a, VT b) {
    if constexpr (OP == DB2_ADD)
        return op_add(a, b);
    else if constexpr (OP == DB2_SUB)
        return op_sub(a, b);
    else if constexpr (OP == DB2_MUL)
        return op_mul(a, b);
    else if constexpr (OP == DB2_DIV)
        return op_div(a, b);
    else if constexpr (OP == DB2_POW)
        return op_pow(a, b);
    else if constexpr (OP == DB2_MOD)
        return op_mod(a, b);
    else if constexpr (OP == DB2_LOG)
        return op_log(a, b);
    else if constexpr (OP == DB2_EQ)
        return (VT)(a == b);
    else if constexpr (OP == DB2_NEQ)
        return (VT)(a != b);
    else if constexpr (OP == DB2_LT)
        return (VT)(a < b);
    else if constexpr (OP == DB2_LE)
        return (VT)(a <= b);
    else if constexpr (OP == DB2_GT)
        return (VT)(a > b);
    else if constexpr (OP == DB2_GE)
        return (VT)(a >= b);
    else if constexpr (OP == DB2_MIN)
        return op_min(a, b);
    else if constexpr (OP == DB2_MAX)
        return op_max(a, b);
    else if constexpr (OP == DB2_AND)
        return (VT)((a != (VT)0) && (b != (VT)0));
    else if constexpr (OP == DB2_OR)
        return (VT)((a != (VT)0) || (b != (VT)0));
    else if constexpr (OP == DB2_BITWISE_AND) {
        if constexpr (std::is_integral_v<VT>)
            return a & b;
        else
            return (VT)((int64_t)a & (int64_t)b);
    } else
        return a;
}

// runtime-opcode form (used by the fused micro-op interpreter; the branch is uniform across the grid)
template <typename VT> __device__ __forceinline__ VT binary_op_rt(int op, VT a, VT b) {
    switch (op) {
    case DB2_ADD: return binary_op<DB2_ADD>(a, b);
    case DB2_SUB: return binary_op<DB2_SUB>(a, b);
    case DB2_MUL: return binary_op<DB2_MUL>(a, b);
    case DB2_DIV: return binary_op<DB2_DIV>(a, b);
    case DB2_POW: return binary_op<DB2_POW>(a, b);
    case DB2_MOD: return binary_op<DB2_MOD>(a, b);
    case DB2_LOG: return binary_op<DB2_LOG>(a, b);
    case DB2_EQ: return binary_op<DB2_EQ>(a, b);
    case DB2_NEQ: return binary_op<DB2_NEQ>(a, b);
    case DB2_LT: return binary_op<DB2_LT>(a, b);
    case DB2_LE: return binary_op<DB2_LE>(a, b);
    case DB2_GT: return binary_op<DB2_GT>(a, b);
    case DB2_GE: return binary_op<DB2_GE>(a, b);
    case DB2_MIN: return binary_op<DB2_MIN>(a, b);
    case DB2_MAX: return binary_op<DB2_MAX>(a, b);
    case DB2_AND: return binary_op<DB2_AND>(a, b);
    case DB2_OR: return binary_op<DB2_OR>(a, b);
    case DB2_BITWISE_AND: return binary_op<DB2_BITWISE_AND>(a, b);
    default: return a;
    }
}

// Unary ops.  `bad` is set when the reference would throw std::domain_error (EwUnarySca.h:134-156,186-195).
template <int OP, typename VT> __device__ __forceinline__ VT unary_op(VT x, bool &bad) {
    // The reference spells the math functions unqualified (sqrt(arg), exp(arg), ...; EwUnarySca.h:186-202), which
    // for float and integer arguments evaluates the C double function and converts the result back; same here.
    using FT = double;
    if constexpr (OP == DB2_U_MINUS) {
        if constexpr (std::is_integral_v<VT>)
            return (VT)(0 - (uint64_t)x);
        else
            return -x;
    } else if constexpr (OP == DB2_U_ABS) {
        if constexpr (std::is_integral_v<VT>)
            return x < 0 ? (VT)(0 - (uint64_t)x) : x;
        else
            return fabs(x);
    } else if constexpr (OP == DB2_U_SIGN) {
        if constexpr (std::is_integral_v<VT>)
            return (x == 0) ? 0 : (x < 0 ? -1 : 1);
        else
            return (x == 0) ? (VT)0 : ((x < 0) ? (VT)-1 : ((x > 0) ? (VT)1 : (VT)NAN));
    } else if constexpr (OP == DB2_U_ISNAN) {
        if constexpr (std::is_integral_v<VT>)
            return 0;
        else
            return (VT)(x != x);
    } else if constexpr (OP == DB2_U_FLOOR) {
        if constexpr (std::is_integral_v<VT>)
            return x;
        else
            return floor(x);
    } else if constexpr (OP == DB2_U_CEIL) {
        if constexpr (std::is_integral_v<VT>)
            return x;
        else
            return ceil(x);
    } else if constexpr (OP == DB2_U_ROUND) {
        if constexpr (std::is_integral_v<VT>)
            return x;
        else
            return round(x);
    } else {
        FT a = (FT)x;
        FT r;
        if constexpr (OP == DB2_U_SQRT) {
            if (a < (FT)0)
                bad = true;
            r = __dsqrt_rn(a);
        } else if constexpr (OP == DB2_U_EXP)
            r = exp(a);
        else if constexpr (OP == DB2_U_LN) {
            if (a < (FT)0)
                bad = true;
            r = log(a);
        } else if constexpr (OP == DB2_U_SIN)
            r = sin(a);
        else if constexpr (OP == DB2_U_COS)
            r = cos(a);
        else if constexpr (OP == DB2_U_TAN)
            r = tan(a);
        else if constexpr (OP == DB2_U_ASIN) {
            if (a < (FT)-1 || a > (FT)1)
                bad = true;
            r = asin(a);
        } else if constexpr (OP == DB2_U_ACOS) {
            if (a < (FT)-1 || a > (FT)1)
                bad = true;
            r = acos(a);
        } else if constexpr (OP == DB2_U_ATAN)
            r = atan(a);
        else if constexpr (OP == DB2_U_SINH)
            r = sinh(a);
        else if constexpr (OP == DB2_U_COSH)
            r = cosh(a);
        else if constexpr (OP == DB2_U_TANH)
            r = tanh(a);
        else
            r = a;
        return (VT)r;
    }
}

template <typename VT> __device__ __forceinline__ VT unary_op_rt(int op, VT x, bool &bad) {
    switch (op) {
    case DB2_U_MINUS: return unary_op<DB2_U_MINUS>(x, bad);
    case DB2_U_ABS: return unary_op<DB2_U_ABS>(x, bad);
    case DB2_U_SIGN: return unary_op<DB2_U_SIGN>(x, bad);
    case DB2_U_SQRT: return unary_op<DB2_U_SQRT>(x, bad);
    case DB2_U_EXP: return unary_op<DB2_U_EXP>(x, bad);
    case DB2_U_LN: return unary_op<DB2_U_LN>(x, bad);
    case DB2_U_SIN: return unary_op<DB2_U_SIN>(x, bad);
    case DB2_U_COS: return unary_op<DB2_U_COS>(x, bad);
    case DB2_U_TAN: return unary_op<DB2_U_TAN>(x, bad);
    case DB2_U_ASIN: return unary_op<DB2_U_ASIN>(x, bad);
    case DB2_U_ACOS: return unary_op<DB2_U_ACOS>(x, bad);
    case DB2_U_ATAN: return unary_op<DB2_U_ATAN>(x, bad);
    case DB2_U_SINH: return unary_op<DB2_U_SINH>(x, bad);
    case DB2_U_COSH: return unary_op<DB2_U_COSH>(x, bad);
    case DB2_U_TANH: return unary_op<DB2_U_TANH>(x, bad);
    case DB2_U_FLOOR: return unary_op<DB2_U_FLOOR>(x, bad);
    case DB2_U_CEIL: return unary_op<DB2_U_CEIL>(x, bad);
    case DB2_U_ROUND: return unary_op<DB2_U_ROUND>(x, bad);
    case DB2_U_ISNAN: return unary_op<DB2_U_ISNAN>(x, bad);
    default: return x;
    }
}

#define DB2_DISPATCH_BINOP(op, OP, ...)                                                                                \
    switch (op) {                                                                                                      \
    case DB2_ADD: { constexpr int OP = DB2_ADD; __VA_ARGS__; } break;                                                  \
    case DB2_SUB: { constexpr int OP = DB2_SUB; __VA_ARGS__; } break;                                                  \
    case DB2_MUL: { constexpr int OP = DB2_MUL; __VA_ARGS__; } break;                                                  \
    case DB2_DIV: { constexpr int OP = DB2_DIV; __VA_ARGS__; } break;                                                  \
    case DB2_POW: { constexpr int OP = DB2_POW; __VA_ARGS__; } break;                                                  \
    case DB2_MOD: { constexpr int OP = DB2_MOD; __VA_ARGS__; } break;                                                  \
    case DB2_LOG: { constexpr int OP = DB2_LOG; __VA_ARGS__; } break;                                                  \
    case DB2_EQ: { constexpr int OP = DB2_EQ; __VA_ARGS__; } break;                                                    \
    case DB2_NEQ: { constexpr int OP = DB2_NEQ; __VA_ARGS__; } break;                                                  \
    case DB2_LT: { constexpr int OP = DB2_LT; __VA_ARGS__; } break;                                                    \
    case DB2_LE: { constexpr int OP = DB2_LE; __VA_ARGS__; } break;                                                    \
    case DB2_GT: { constexpr int OP = DB2_GT; __VA_ARGS__; } break;                                                    \
    case DB2_GE: { constexpr int OP = DB2_GE; __VA_ARGS__; } break;                                                    \
    case DB2_MIN: { constexpr int OP = DB2_MIN; __VA_ARGS__; } break;                                                  \
    case DB2_MAX: { constexpr int OP = DB2_MAX; __VA_ARGS__; } break;                                                  \
    case DB2_AND: { constexpr int OP = DB2_AND; __VA_ARGS__; } break;                                                  \
    case DB2_OR: { constexpr int OP = DB2_OR; __VA_ARGS__; } break;                                                    \
    case DB2_BITWISE_AND: { constexpr int OP = DB2_BITWISE_AND; __VA_ARGS__; } break;                                  \
    default:                                                                                                           \
        return ::db2::set_error(DB2_EUNSUPPORTED, "unknown BinaryOpCode %d", (int)(op));                               \
    }

#define DB2_DISPATCH_UNOP(op, OP, ...)                                                                                 \
    switch (op) {                                                                                                      \
    case DB2_U_MINUS: { constexpr int OP = DB2_U_MINUS; __VA_ARGS__; } break;                                          \
    case DB2_U_ABS: { constexpr int OP = DB2_U_ABS; __VA_ARGS__; } break;                                              \
    case DB2_U_SIGN: { constexpr int OP = DB2_U_SIGN; __VA_ARGS__; } break;                                            \
    case DB2_U_SQRT: { constexpr int OP = DB2_U_SQRT; __VA_ARGS__; } break;                                            \
    case DB2_U_EXP: { constexpr int OP = DB2_U_EXP; __VA_ARGS__; } break;                                              \
    case DB2_U_LN: { constexpr int OP = DB2_U_LN; __VA_ARGS__; } break;                                                \
    case DB2_U_SIN: { constexpr int OP = DB2_U_SIN; __VA_ARGS__; } break;                                              \
    case DB2_U_COS: { constexpr int OP = DB2_U_COS; __VA_ARGS__; } break;                                              \
    case DB2_U_TAN: { constexpr int OP = DB2_U_TAN; __VA_ARGS__; } break;                                              \
    case DB2_U_ASIN: { constexpr int OP = DB2_U_ASIN; __VA_ARGS__; } break;                                            \
    case DB2_U_ACOS: { constexpr int OP = DB2_U_ACOS; __VA_ARGS__; } break;                                            \
    case DB2_U_ATAN: { constexpr int OP = DB2_U_ATAN; __VA_ARGS__; } break;                                            \
    case DB2_U_SINH: { constexpr int OP = DB2_U_SINH; __VA_ARGS__; } break;                                            \
    case DB2_U_COSH: { constexpr int OP = DB2_U_COSH; __VA_ARGS__; } break;                                            \
    case DB2_U_TANH: { constexpr int OP = DB2_U_TANH; __VA_ARGS__; } break;                                            \
    case DB2_U_FLOOR: { constexpr int OP = DB2_U_FLOOR; __VA_ARGS__; } break;                                          \
    case DB2_U_CEIL: { constexpr int OP = DB2_U_CEIL; __VA_ARGS__; } break;                                            \
    case DB2_U_ROUND: { constexpr int OP = DB2_U_ROUND; __VA_ARGS__; } break;                                          \
    case DB2_U_ISNAN: { constexpr int OP = DB2_U_ISNAN; __VA_ARGS__; } break;                                          \
    default:                                                                                                           \
        return ::db2::set_error(DB2_EUNSUPPORTED, "unknown UnaryOpCode %d", (int)(op));                                \
    }

} // namespace db2
