/*
 * TEST INFRASTRUCTURE -- not part of the product.
 *
 * Plain-C restatement of the CPU kernels of DAPHNE (daphne-eu/daphne, src/runtime/local/kernels) that the CUDA
 * library in daphne_b200/ replaces.  It exists only as the checker for tests/, for __graft_entry__.smoke() and for
 * the cpu_baseline leg of bench.py; nothing in daphne_b200/ may call it.
 *
 * Every function walks the data in the same order and with the same scalar expressions as the reference function it
 * cites, so that floating-point results carry the same rounding as the reference's CPU kernels built with gcc at
 * -O2 without -ffast-math (this file must be compiled with -ffp-contract=off so that no a*b+c is fused).
 * Pinned against: the literal expected values of the reference's unit tests (tests/golden/*.json, taken from
 * test/runtime/local/kernels/{AggRow,AggCol,AggAll,EwBinaryMat,EwBinaryObjSca,EwUnaryMat,Syrk,MatMul,Gemv,Solve,
 * CTable,Transpose}Test.cpp) and against the reference's own kernels compiled from its sources (oracle/_ref,
 * tests/test_oracle_vs_ref.py).
 *
 * Conventions: row-major, leading dimension in elements, op codes = the reference's enum values
 * (BinaryOpCode.h:29-56, UnaryOpCode.h:26-56, AggOpCode.h:25-35).  Return 0 = ok, 1 = invalid argument
 * (the reference throws std::runtime_error), 5 = domain error (std::domain_error).
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

enum { ADD = 0, SUB, MUL, DIV, POW, MOD, LOG, EQ, NEQ, LT, LE, GT, GE, MIN, MAX, AND, OR, BITWISE_AND };
enum { U_MINUS = 0, U_ABS, U_SIGN, U_SQRT, U_EXP, U_LN, U_SIN, U_COS, U_TAN, U_ASIN, U_ACOS, U_ATAN, U_SINH, U_COSH,
       U_TANH, U_FLOOR, U_CEIL, U_ROUND, U_ISNAN };
enum { A_SUM = 0, A_PROD, A_MIN, A_MAX, A_IDXMIN, A_IDXMAX, A_MEAN, A_STDDEV, A_VAR };

/* ------------------------------------------------------------------------------------------------------------- */
/* scalar ops: EwBinarySca.h:138-166 (MAKE_EW_BINARY_SCA lines)                                                   */
/* ------------------------------------------------------------------------------------------------------------- */
#define DEF_BIN(NAME, VT)                                                                                              \
    static VT bin_##NAME(int op, VT a, VT b) {                                                                         \
        switch (op) {                                                                                                  \
        case ADD: return a + b;                                                                                        \
        case SUB: return a - b;                                                                                        \
        case MUL: return a * b;                                                                                        \
        case DIV: return a / b;                                                                                        \
        case POW: return (VT)pow((double)a, (double)b);                                                                \
        case MOD: return (VT)fmod((double)a, (double)b);                                                               \
        case LOG: return (VT)(log((double)a) / log((double)b));                                                        \
        case EQ: return (VT)(a == b);                                                                                  \
        case NEQ: return (VT)(a != b);                                                                                 \
        case LT: return (VT)(a < b);                                                                                   \
        case LE: return (VT)(a <= b);                                                                                  \
        case GT: return (VT)(a > b);                                                                                   \
        case GE: return (VT)(a >= b);                                                                                  \
        case MIN: return (b < a) ? b : a; /* std::min */                                                               \
        case MAX: return (a < b) ? b : a; /* std::max */                                                               \
        case AND: return (VT)(a && b);                                                                                 \
        case OR: return (VT)(a || b);                                                                                  \
        case BITWISE_AND: return (VT)((int64_t)a & (int64_t)b);                                                        \
        default: return a;                                                                                             \
        }                                                                                                              \
    }
DEF_BIN(f64, double)
DEF_BIN(i64, int64_t)
/* the other integer value types of EwBinaryMat / EwBinaryObjSca (kernels.json: uint64_t, int32_t, uint32_t); pow, fmod
 * and log promote the integer operands to double as the unqualified calls in the reference do */
DEF_BIN(u64, uint64_t)
DEF_BIN(i32, int32_t)
DEF_BIN(u32, uint32_t)
/* float: fmodf / logf are what std::fmod(float,float) and std::log(float) resolve to */
static float bin_f32(int op, float a, float b) {
    switch (op) {
    case ADD: return a + b;
    case SUB: return a - b;
    case MUL: return a * b;
    case DIV: return a / b;
    case POW: return (float)pow((double)a, (double)b);
    case MOD: return fmodf(a, b);
    case LOG: return logf(a) / logf(b);
    case EQ: return (float)(a == b);
    case NEQ: return (float)(a != b);
    case LT: return (float)(a < b);
    case LE: return (float)(a <= b);
    case GT: return (float)(a > b);
    case GE: return (float)(a >= b);
    case MIN: return (b < a) ? b : a;
    case MAX: return (a < b) ? b : a;
    case AND: return (float)(a && b);
    case OR: return (float)(a || b);
    default: return a;
    }
}

/* EwUnarySca.h:182-206; *bad is set where the reference throws std::domain_error (:134-156) */
static double un_f64(int op, double x, int *bad) {
    switch (op) {
    case U_MINUS: return -x;
    case U_ABS: return fabs(x);
    case U_SIGN: return (x == 0) ? 0 : ((x < 0) ? -1 : ((x > 0) ? 1 : NAN));
    case U_SQRT: if (-0.0 > x) *bad = 1; return sqrt(x);
    case U_EXP: return exp(x);
    case U_LN: if (-0.0 > x) *bad = 1; return log(x);
    case U_SIN: return sin(x);
    case U_COS: return cos(x);
    case U_TAN: return tan(x);
    case U_ASIN: if (-1.0 > x || x > 1.0) *bad = 1; return asin(x);
    case U_ACOS: if (-1.0 > x || x > 1.0) *bad = 1; return acos(x);
    case U_ATAN: return atan(x);
    case U_SINH: return sinh(x);
    case U_COSH: return cosh(x);
    case U_TANH: return tanh(x);
    case U_FLOOR: return floor(x);
    case U_CEIL: return ceil(x);
    case U_ROUND: return round(x);
    case U_ISNAN: return (double)(x != x);
    default: return x;
    }
}
/* float: the reference spells most functions unqualified (sqrt(arg), exp(arg), sin(arg), ...), which binds to the C
 * double functions, and rounds the double result to float; only std::abs and std::ceil use the float overloads. */
static float un_f32(int op, float x, int *bad) {
    switch (op) {
    case U_MINUS: return -x;
    case U_ABS: return fabsf(x);
    case U_SIGN: return (x == 0) ? 0 : ((x < 0) ? -1 : ((x > 0) ? 1 : NAN));
    case U_CEIL: return ceilf(x);
    case U_ISNAN: return (float)(x != x);
    default: return (float)un_f64(op, (double)x, bad);
    }
}
static int64_t un_i64(int op, int64_t x, int *bad) {
    switch (op) {
    case U_MINUS: return -x;
    case U_ABS: return x < 0 ? -x : x;
    case U_SIGN: return (x == 0) ? 0 : ((x < 0) ? -1 : 1);
    case U_FLOOR: case U_CEIL: case U_ROUND: return x;
    case U_ISNAN: return 0;
    default: return (int64_t)un_f64(op, (double)x, bad);
    }
}

/* ------------------------------------------------------------------------------------------------------------- */
/* EwBinaryMat<Dense,Dense,Dense>  (EwBinaryMat.h:54-108)                                                         */
/* ------------------------------------------------------------------------------------------------------------- */
#define DEF_EW_BINARY(NAME, VT)                                                                                        \
    int orc_ew_binary_##NAME(int op, const VT *lhs, int64_t lr, int64_t lc, int64_t lld, const VT *rhs, int64_t rr,    \
                             int64_t rc, int64_t rld, VT *res, int64_t res_ld) {                                       \
        if (lr == rr && lc == rc) {                                                                                    \
            for (int64_t r = 0; r < lr; r++)                                                                           \
                for (int64_t c = 0; c < lc; c++)                                                                       \
                    res[r * res_ld + c] = bin_##NAME(op, lhs[r * lld + c], rhs[r * rld + c]);                          \
        } else if (lc == rc && (rr == 1 || lr == 1)) {                                                                 \
            for (int64_t r = 0; r < lr; r++)                                                                           \
                for (int64_t c = 0; c < lc; c++)                                                                       \
                    res[r * res_ld + c] = bin_##NAME(op, lhs[r * lld + c], rhs[c]);                                    \
        } else if (lr == rr && (rc == 1 || lc == 1)) {                                                                 \
            for (int64_t r = 0; r < lr; r++)                                                                           \
                for (int64_t c = 0; c < lc; c++)                                                                       \
                    res[r * res_ld + c] = bin_##NAME(op, lhs[r * lld + c], rhs[r * rld]);                              \
        } else                                                                                                         \
            return 1;                                                                                                  \
        return 0;                                                                                                      \
    }                                                                                                                  \
    /* EwBinaryObjSca<Dense,Dense,VT> (EwBinaryObjSca.h:58-79) */                                                      \
    int orc_ew_binary_sca_##NAME(int op, const VT *lhs, int64_t rows, int64_t cols, int64_t ld, VT s, VT *res,         \
                                 int64_t res_ld) {                                                                     \
        for (int64_t r = 0; r < rows; r++)                                                                             \
            for (int64_t c = 0; c < cols; c++)                                                                         \
                res[r * res_ld + c] = bin_##NAME(op, lhs[r * ld + c], s);                                              \
        return 0;                                                                                                      \
    }                                                                                                                  \
    /* EwUnaryMat<Dense,Dense> (EwUnaryMat.h:57-77) */                                                                 \
    int orc_ew_unary_##NAME(int op, const VT *arg, int64_t rows, int64_t cols, int64_t ld, VT *res, int64_t res_ld) {  \
        int bad = 0;                                                                                                   \
        for (int64_t r = 0; r < rows; r++)                                                                             \
            for (int64_t c = 0; c < cols; c++)                                                                         \
                res[r * res_ld + c] = un_##NAME(op, arg[r * ld + c], &bad);                                            \
        return bad ? 5 : 0;                                                                                            \
    }
DEF_EW_BINARY(f64, double)
DEF_EW_BINARY(f32, float)
DEF_EW_BINARY(i64, int64_t)
/* binary forms only (no unary kernel is instantiated for these value types) */
static uint64_t un_u64(int op, uint64_t x, int *bad) { (void)op; (void)bad; return x; }
static int32_t un_i32(int op, int32_t x, int *bad) { (void)op; (void)bad; return x; }
static uint32_t un_u32(int op, uint32_t x, int *bad) { (void)op; (void)bad; return x; }
DEF_EW_BINARY(u64, uint64_t)
DEF_EW_BINARY(i32, int32_t)
DEF_EW_BINARY(u32, uint32_t)

/* ------------------------------------------------------------------------------------------------------------- */
/* aggregations                                                                                                   */
/* ------------------------------------------------------------------------------------------------------------- */
#define NEUTRAL_MIN_f64 INFINITY
#define NEUTRAL_MAX_f64 (-INFINITY)
#define NEUTRAL_MIN_f32 INFINITY
#define NEUTRAL_MAX_f32 (-INFINITY)
#define NEUTRAL_MIN_i64 INT64_MAX
#define NEUTRAL_MAX_i64 INT64_MIN
#define SQRT_f64(x) sqrt(x)
#define SQRT_f32(x) ((float)sqrt(x)) /* unqualified sqrt(float) in the reference binds to the double overload set */
#define SQRT_i64(x) ((int64_t)sqrt((double)(x)))

static int agg_bin_op(int op) {
    switch (op) {
    case A_SUM: case A_MEAN: case A_STDDEV: case A_VAR: return ADD;
    case A_PROD: return MUL;
    case A_MIN: return MIN;
    case A_MAX: return MAX;
    default: return -1;
    }
}

#define DEF_AGG(NAME, VT)                                                                                              \
    /* AggRow<Dense,Dense> (AggRow.h:60-161).  idx results go to res_idx (uint64), others to res. */                   \
    int orc_agg_row_##NAME(int op, const VT *arg, int64_t rows, int64_t cols, int64_t ld, VT *res, uint64_t *res_idx,  \
                           int64_t res_ld) {                                                                           \
        if (op == A_IDXMIN || op == A_IDXMAX) {                                                                        \
            for (int64_t r = 0; r < rows; r++) {                                                                       \
                const VT *row = arg + r * ld;                                                                          \
                VT best = row[0];                                                                                      \
                uint64_t idx = 0;                                                                                      \
                for (int64_t c = 1; c < cols; c++)                                                                     \
                    if (op == A_IDXMIN ? (row[c] < best) : (row[c] > best)) {                                          \
                        best = row[c];                                                                                 \
                        idx = (uint64_t)c;                                                                             \
                    }                                                                                                  \
                res_idx[r * res_ld] = idx;                                                                             \
            }                                                                                                          \
            return 0;                                                                                                  \
        }                                                                                                              \
        const int bop = agg_bin_op(op);                                                                                \
        if (bop < 0)                                                                                                   \
            return 1;                                                                                                  \
        for (int64_t r = 0; r < rows; r++) {                                                                           \
            const VT *row = arg + r * ld;                                                                              \
            VT agg = row[0];                                                                                           \
            for (int64_t c = 1; c < cols; c++)                                                                         \
                agg = bin_##NAME(bop, agg, row[c]);                                                                    \
            res[r * res_ld] = agg;                                                                                     \
        }                                                                                                              \
        if (op == A_SUM || op == A_PROD || op == A_MIN || op == A_MAX)                                                 \
            return 0;                                                                                                  \
        for (int64_t r = 0; r < rows; r++)                                                                             \
            res[r * res_ld] = (VT)(res[r * res_ld] / (size_t)cols);                                                    \
        if (op == A_MEAN)                                                                                              \
            return 0;                                                                                                  \
        for (int64_t r = 0; r < rows; r++) {                                                                           \
            const VT *row = arg + r * ld;                                                                              \
            VT t = 0;                                                                                                  \
            for (int64_t c = 0; c < cols; c++) {                                                                       \
                VT val = row[c] - res[r * res_ld];                                                                     \
                t = t + val * val;                                                                                     \
            }                                                                                                          \
            t = (VT)(t / (size_t)cols);                                                                                \
            res[r * res_ld] = (op == A_STDDEV) ? SQRT_##NAME(t) : t;                                                   \
        }                                                                                                              \
        return 0;                                                                                                      \
    }                                                                                                                  \
    /* AggCol<Dense,Dense> (AggCol.h:58-178) */                                                                        \
    int orc_agg_col_##NAME(int op, const VT *arg, int64_t rows, int64_t cols, int64_t ld, VT *res,                     \
                           uint64_t *res_idx) {                                                                        \
        if (op == A_IDXMIN || op == A_IDXMAX) {                                                                        \
            VT *tmp = (VT *)malloc(sizeof(VT) * (size_t)(cols ? cols : 1));                                            \
            memcpy(tmp, arg, sizeof(VT) * (size_t)cols);                                                               \
            for (int64_t c = 0; c < cols; c++)                                                                         \
                res_idx[c] = 0;                                                                                        \
            for (int64_t r = 1; r < rows; r++)                                                                         \
                for (int64_t c = 0; c < cols; c++) {                                                                   \
                    const VT x = arg[r * ld + c];                                                                      \
                    if (op == A_IDXMIN ? (x < tmp[c]) : (x > tmp[c])) {                                                \
                        tmp[c] = x;                                                                                    \
                        res_idx[c] = (uint64_t)r;                                                                      \
                    }                                                                                                  \
                }                                                                                                      \
            free(tmp);                                                                                                 \
            return 0;                                                                                                  \
        }                                                                                                              \
        const int bop = agg_bin_op(op);                                                                                \
        if (bop < 0)                                                                                                   \
            return 1;                                                                                                  \
        for (int64_t c = 0; c < cols; c++)                                                                             \
            res[c] = arg[c];                                                                                           \
        for (int64_t r = 1; r < rows; r++)                                                                             \
            for (int64_t c = 0; c < cols; c++)                                                                         \
                res[c] = bin_##NAME(bop, res[c], arg[r * ld + c]);                                                     \
        if (op == A_SUM || op == A_PROD || op == A_MIN || op == A_MAX)                                                 \
            return 0;                                                                                                  \
        for (int64_t c = 0; c < cols; c++)                                                                             \
            res[c] = (VT)(res[c] / (size_t)rows);                                                                      \
        if (op == A_MEAN)                                                                                              \
            return 0;                                                                                                  \
        VT *t = (VT *)calloc((size_t)(cols ? cols : 1), sizeof(VT));                                                   \
        for (int64_t r = 0; r < rows; r++)                                                                             \
            for (int64_t c = 0; c < cols; c++) {                                                                       \
                VT val = arg[r * ld + c] - res[c];                                                                     \
                t[c] = t[c] + val * val;                                                                               \
            }                                                                                                          \
        for (int64_t c = 0; c < cols; c++) {                                                                           \
            t[c] = (VT)(t[c] / (size_t)rows);                                                                          \
            if (op == A_STDDEV)                                                                                        \
                t[c] = SQRT_##NAME(t[c]);                                                                              \
        }                                                                                                              \
        memcpy(res, t, sizeof(VT) * (size_t)cols);                                                                     \
        free(t);                                                                                                       \
        return 0;                                                                                                      \
    }                                                                                                                  \
    /* aggAllArray (AggAll.h:64-96): four interleaved accumulators, pairwise fold, then the tail */                    \
    static VT agg_all_array_##NAME(int bop, const VT *v, size_t n, VT neutral) {                                       \
        VT agg;                                                                                                        \
        if (n) {                                                                                                       \
            VT a0 = neutral, a1 = neutral, a2 = neutral, a3 = neutral;                                                 \
            for (size_t i = 0; i < n / 4 * 4; i += 4) {                                                                \
                a0 = bin_##NAME(bop, a0, v[i]);                                                                        \
                a1 = bin_##NAME(bop, a1, v[i + 1]);                                                                    \
                a2 = bin_##NAME(bop, a2, v[i + 2]);                                                                    \
                a3 = bin_##NAME(bop, a3, v[i + 3]);                                                                    \
            }                                                                                                          \
            agg = bin_##NAME(bop, bin_##NAME(bop, a0, a1), bin_##NAME(bop, a2, a3));                                   \
            for (size_t i = 0; i < n % 4; i++)                                                                         \
                agg = bin_##NAME(bop, agg, v[n / 4 * 4 + i]);                                                          \
        } else                                                                                                         \
            agg = neutral;                                                                                             \
        return agg;                                                                                                    \
    }                                                                                                                  \
    /* AggAll<VT,Dense> (AggAll.h:124-193) */                                                                          \
    int orc_agg_all_##NAME(int op, const VT *arg, int64_t rows, int64_t cols, int64_t ld, VT *res) {                   \
        const int bop = agg_bin_op(op);                                                                                \
        if (bop < 0)                                                                                                   \
            return 1;                                                                                                  \
        VT neutral = 0;                                                                                                \
        if (op == A_PROD) neutral = 1;                                                                                 \
        if (op == A_MIN) neutral = NEUTRAL_MIN_##NAME;                                                                 \
        if (op == A_MAX) neutral = NEUTRAL_MAX_##NAME;                                                                 \
        VT agg;                                                                                                        \
        if (cols == ld || rows == 1)                                                                                   \
            agg = agg_all_array_##NAME(bop, arg, (size_t)(rows * cols), neutral);                                      \
        else {                                                                                                         \
            agg = neutral;                                                                                             \
            for (int64_t r = 0; r < rows; r++)                                                                         \
                agg = bin_##NAME(bop, agg, agg_all_array_##NAME(bop, arg + r * ld, (size_t)cols, neutral));            \
        }                                                                                                              \
        if (op == A_SUM || op == A_PROD || op == A_MIN || op == A_MAX) {                                               \
            *res = agg;                                                                                                \
            return 0;                                                                                                  \
        }                                                                                                              \
        agg = (VT)(agg / ((size_t)cols * (size_t)rows));                                                               \
        if (op == A_MEAN) {                                                                                            \
            *res = agg;                                                                                                \
            return 0;                                                                                                  \
        }                                                                                                              \
        VT sd = 0;                                                                                                     \
        for (int64_t r = 0; r < rows; r++)                                                                             \
            for (int64_t c = 0; c < cols; c++) {                                                                       \
                VT val = arg[r * ld + c] - agg;                                                                        \
                sd = sd + val * val;                                                                                   \
            }                                                                                                          \
        sd = (VT)(sd / ((size_t)cols * (size_t)rows));                                                                 \
        *res = (op == A_VAR) ? sd : SQRT_##NAME(sd);                                                                   \
        return 0;                                                                                                      \
    }
DEF_AGG(f64, double)
DEF_AGG(f32, float)
DEF_AGG(i64, int64_t)

/* ------------------------------------------------------------------------------------------------------------- */
/* contractions and helpers                                                                                       */
/* ------------------------------------------------------------------------------------------------------------- */
/* MatMul<Dense,Dense,Dense> (MatMul.cpp:248-290).  The reference hands the arithmetic to OpenBLAS (cblas_ddot /
 * cblas_dgemv / cblas_dgemm, a third-party dependency pinned to 0.3.23 in software-package-versions.txt:27 and not
 * part of the reference tree); BLAS fixes no summation order, so this restatement is the textbook triple loop and
 * parity for the contractions is a tolerance statement (relative to the largest entry of the result), pinned by the
 * exact small integer cases of MatMulTest.cpp / SyrkTest.cpp. */
int orc_matmul_f64(const double *a, int64_t ar, int64_t ac, int64_t lda, const double *b, int64_t br, int64_t bc,
                   int64_t ldb, int transa, int transb, double *res, int64_t ldc) {
    const int64_t m = transa ? ac : ar, k = transa ? ar : ac, k2 = transb ? bc : br, n = transb ? br : bc;
    if (k != k2)
        return 1;
    for (int64_t i = 0; i < m; i++)
        for (int64_t j = 0; j < n; j++) {
            double s = 0.0;
            for (int64_t l = 0; l < k; l++) {
                const double x = transa ? a[l * lda + i] : a[i * lda + l];
                const double y = transb ? b[j * ldb + l] : b[l * ldb + j];
                s = s + x * y;
            }
            res[i * ldc + j] = s;
        }
    return 0;
}

/* MatMul for int64_t / int32_t (MatMul.cpp:40-57, 78-134 and the gemm specialisations below them: Eigen products, a
 * third-party dependency that is not part of the reference tree).  Integer products and sums wrap and are associative,
 * so every evaluation order gives these bits; the arithmetic is done on the unsigned type to stay defined. */
int orc_matmul_i64(const int64_t *a, int64_t ar, int64_t ac, int64_t lda, const int64_t *b, int64_t br, int64_t bc,
                   int64_t ldb, int transa, int transb, int64_t *res, int64_t ldc) {
    const int64_t m = transa ? ac : ar, k = transa ? ar : ac, k2 = transb ? bc : br, n = transb ? br : bc;
    if (k != k2)
        return 1;
    for (int64_t i = 0; i < m; i++)
        for (int64_t j = 0; j < n; j++) {
            uint64_t s = 0;
            for (int64_t l = 0; l < k; l++) {
                const uint64_t x = (uint64_t)(transa ? a[l * lda + i] : a[i * lda + l]);
                const uint64_t y = (uint64_t)(transb ? b[j * ldb + l] : b[l * ldb + j]);
                s += x * y;
            }
            res[i * ldc + j] = (int64_t)s;
        }
    return 0;
}
int orc_matmul_i32(const int32_t *a, int64_t ar, int64_t ac, int64_t lda, const int32_t *b, int64_t br, int64_t bc,
                   int64_t ldb, int transa, int transb, int32_t *res, int64_t ldc) {
    const int64_t m = transa ? ac : ar, k = transa ? ar : ac, k2 = transb ? bc : br, n = transb ? br : bc;
    if (k != k2)
        return 1;
    for (int64_t i = 0; i < m; i++)
        for (int64_t j = 0; j < n; j++) {
            uint32_t s = 0;
            for (int64_t l = 0; l < k; l++) {
                const uint32_t x = (uint32_t)(transa ? a[l * lda + i] : a[i * lda + l]);
                const uint32_t y = (uint32_t)(transb ? b[j * ldb + l] : b[l * ldb + j]);
                s += x * y;
            }
            res[i * ldc + j] = (int32_t)s;
        }
    return 0;
}
/* Syrk<Dense,Dense> (Syrk.h:51-71): cblas_dsyrk on the upper triangle, then the mirror loop (:65-69) */
int orc_syrk_f64(const double *arg, int64_t rows, int64_t cols, int64_t ld, int trans_left, double *res) {
    const int64_t n = trans_left ? cols : rows, k = trans_left ? rows : cols;
    for (int64_t i = 0; i < n; i++)
        for (int64_t j = i; j < n; j++) {
            double s = 0.0;
            for (int64_t l = 0; l < k; l++) {
                const double x = trans_left ? arg[l * ld + i] : arg[i * ld + l];
                const double y = trans_left ? arg[l * ld + j] : arg[j * ld + l];
                s = s + x * y;
            }
            res[i * n + j] = s;
        }
    for (int64_t r = 0; r < n; r++)
        for (int64_t c = r + 1; c < n; c++)
            res[c * n + r] = res[r * n + c];
    return 0;
}
/* Gemv<Dense,Dense,Dense> (Gemv.h:51-63): res = t(mat) vec */
int orc_gemv_f64(const double *mat, int64_t rows, int64_t cols, int64_t ld, const double *vec, int64_t vec_ld,
                 double *res) {
    for (int64_t c = 0; c < cols; c++)
        res[c] = 0.0;
    for (int64_t r = 0; r < rows; r++)
        for (int64_t c = 0; c < cols; c++)
            res[c] = res[c] + mat[r * ld + c] * vec[r * vec_ld];
    return 0;
}
/* Solve<Dense,Dense,Dense> (Solve.h:86-116): LAPACKE_dgesv = LU with partial pivoting (first largest |a_ik| as
 * pivot, like idamax) followed by forward and back substitution.  Returns 1 when a pivot is exactly zero (the
 * reference throws "A factor Ui is exactly singular"). */
int orc_solve_f64(const double *a, int64_t n, const double *b, double *x) {
    double *w = (double *)malloc(sizeof(double) * (size_t)(n * n ? n * n : 1));
    memcpy(w, a, sizeof(double) * (size_t)(n * n));
    memcpy(x, b, sizeof(double) * (size_t)n);
    for (int64_t k = 0; k < n; k++) {
        int64_t piv = k;
        double best = fabs(w[k * n + k]);
        for (int64_t i = k + 1; i < n; i++)
            if (fabs(w[i * n + k]) > best) {
                best = fabs(w[i * n + k]);
                piv = i;
            }
        if (best == 0.0) {
            free(w);
            return 1;
        }
        if (piv != k) {
            for (int64_t c = 0; c < n; c++) {
                double t = w[k * n + c];
                w[k * n + c] = w[piv * n + c];
                w[piv * n + c] = t;
            }
            double t = x[k];
            x[k] = x[piv];
            x[piv] = t;
        }
        for (int64_t i = k + 1; i < n; i++) {
            const double l = w[i * n + k] / w[k * n + k];
            w[i * n + k] = l;
            for (int64_t j = k + 1; j < n; j++)
                w[i * n + j] = w[i * n + j] - l * w[k * n + j];
            x[i] = x[i] - l * x[k];
        }
    }
    for (int64_t k = n - 1; k >= 0; k--) {
        x[k] = x[k] / w[k * n + k];
        for (int64_t i = 0; i < k; i++)
            x[i] = x[i] - w[i * n + k] * x[k];
    }
    free(w);
    return 0;
}
/* Transpose<Dense,Dense> (Transpose.h:51-76) */
int orc_transpose_f64(const double *arg, int64_t rows, int64_t cols, int64_t ld, double *res) {
    for (int64_t r = 0; r < rows; r++)
        for (int64_t c = 0; c < cols; c++)
            res[c * rows + r] = arg[r * ld + c];
    return 0;
}
/* CTable<Dense<double>,Dense<int64>,Dense<int64>,double> (CTable.h:55-106).  res_rows / res_cols < 0: derived from the
 * largest coordinate; res must then be sized by the caller after a first call with res == NULL. */
int orc_ctable_f64(const int64_t *lhs, const int64_t *rhs, int64_t n, double weight, int64_t res_rows,
                   int64_t res_cols, double *res, int64_t *out_rows, int64_t *out_cols) {
    const int rows_from_lhs = res_rows < 0, cols_from_rhs = res_cols < 0;
    if (rows_from_lhs) {
        int64_t m = lhs[0];
        for (int64_t i = 1; i < n; i++)
            if (lhs[i] > m) m = lhs[i];
        res_rows = m + 1;
    }
    if (cols_from_rhs) {
        int64_t m = rhs[0];
        for (int64_t i = 1; i < n; i++)
            if (rhs[i] > m) m = rhs[i];
        res_cols = m + 1;
    }
    *out_rows = res_rows;
    *out_cols = res_cols;
    if (!res)
        return 0;
    memset(res, 0, sizeof(double) * (size_t)(res_rows * res_cols));
    for (int64_t i = 0; i < n; i++) {
        const int64_t r = lhs[i], c = rhs[i];
        if ((rows_from_lhs && cols_from_rhs) || (r < res_rows && c < res_cols))
            res[r * res_cols + c] += weight;
    }
    return 0;
}
/* Seq<Dense<double>> (Seq.h:49-99): repeated addition of inc, then the end-point trim */
int orc_seq_f64(double start, double end, double inc, double *res, int64_t cap, int64_t *n_out) {
    if (inc != inc || start != start || end != end || inc == 0)
        return 1;
    if ((start < end && inc < 0) || (start > end && inc > 0)) {
        *n_out = 0;
        return 0;
    }
    const int64_t expected = (int64_t)ceil(fabs(end - start) / fabs(inc)) + 1;
    double acc = start, last = start;
    for (int64_t i = 0; i < expected; i++) {
        if (res && i < cap)
            res[i] = acc;
        last = acc;
        acc += inc;
    }
    int64_t n = expected;
    const double eps = 1.0e-13;
    if ((end < start) && end - last > eps)
        n--;
    else if ((end > start) && last - end > eps)
        n--;
    *n_out = n;
    return 0;
}

/* ------------------------------------------------------------------------------------------------------------- */
/* CSR kernels (values double, indices size_t as in CSRMatrix.h:70-72)                                            */
/* ------------------------------------------------------------------------------------------------------------- */
/* EwBinaryMat<CSR,CSR,Dense> for MUL (EwBinaryMat.h:254-317): rhs has the shape of lhs or is a row/column vector;
 * entries where rhs is exactly 0 are dropped.  Outputs sized for nnz(lhs). */
int orc_csr_ewmul_dense_f64(const double *vals, const uint64_t *cidx, const uint64_t *roff, int64_t rows, int64_t cols,
                            const double *rhs, int64_t rr, int64_t rc, double *ovals, uint64_t *ocidx, uint64_t *oroff,
                            int64_t *out_nnz) {
    if ((rows != rr && rr != 1) || (cols != rc && rc != 1))
        return 1;
    oroff[0] = 0;
    for (int64_t r = 0; r < rows; r++) {
        uint64_t pos = oroff[r];
        const int64_t rhs_row = (rr == 1) ? 0 : r;
        for (uint64_t i = roff[r]; i < roff[r + 1]; i++) {
            const int64_t rhs_col = (rc == 1) ? 0 : (int64_t)cidx[i];
            const double rv = rhs[rhs_row * rc + rhs_col];
            if (rv != 0) {
                ovals[pos] = vals[i] * rv;
                ocidx[pos] = cidx[i];
                pos++;
            }
        }
        oroff[r + 1] = pos;
    }
    *out_nnz = (int64_t)oroff[rows];
    return 0;
}
/* AggRow<Dense,CSR> (AggRow.h:178-238) for the pure reductions: aggAllArray over the row's stored values, then one
 * implicit zero if the op is not sparse-safe and the row is not full (AggOpCode.h:84-100). */
int orc_csr_agg_row_f64(int op, const double *vals, const uint64_t *roff, int64_t rows, int64_t cols, double *res) {
    const int bop = agg_bin_op(op);
    if (bop < 0 || op == A_MEAN || op == A_STDDEV || op == A_VAR)
        return 1;
    double neutral = 0;
    if (op == A_PROD) neutral = 1;
    if (op == A_MIN) neutral = INFINITY;
    if (op == A_MAX) neutral = -INFINITY;
    const int sparse_safe = (op == A_SUM);
    for (int64_t r = 0; r < rows; r++) {
        const size_t n = (size_t)(roff[r + 1] - roff[r]);
        double agg = agg_all_array_f64(bop, vals + roff[r], n, neutral);
        if (!sparse_safe && (int64_t)n < cols)
            agg = bin_f64(bop, agg, 0);
        res[r] = agg;
    }
    return 0;
}
/* Gemv<Dense,CSR,Dense> (Gemv.h:79-117): res = mat @ vec for a dense vec with vcols columns */
int orc_csr_gemv_f64(const double *vals, const uint64_t *cidx, const uint64_t *roff, int64_t rows, const double *vec,
                     int64_t vcols, double *res) {
    memset(res, 0, sizeof(double) * (size_t)(rows * vcols));
    for (int64_t r = 0; r < rows; r++)
        for (uint64_t i = roff[r]; i < roff[r + 1]; i++)
            for (int64_t j = 0; j < vcols; j++)
                res[r * vcols + j] += vals[i] * vec[(int64_t)cidx[i] * vcols + j];
    return 0;
}
