// TEST INFRASTRUCTURE -- not part of the product.
//
// Plain-C entry points over the REAL CPU kernels of a DAPHNE source tree (the headers are included from
// $DAPHNE_SRC/src, nothing of them is copied here).  Built by oracle/Makefile into oracle/_ref/libdaphne_ref.so and
// used (a) to validate the C restatement in oracle.c and (b) as the "reference" CPU baseline of bench.py.
// The signatures are those of the orc_* functions in oracle.c with the prefix ref_.
#include <runtime/local/datastructures/CSRMatrix.h>
#include <runtime/local/datastructures/DataObjectFactory.h>
#include <runtime/local/datastructures/DenseMatrix.h>
#include <runtime/local/kernels/AggAll.h>
#include <runtime/local/kernels/AggCol.h>
#include <runtime/local/kernels/AggRow.h>
#include <runtime/local/kernels/CTable.h>
#include <runtime/local/kernels/EwBinaryMat.h>
#include <runtime/local/kernels/EwBinaryObjSca.h>
#include <runtime/local/kernels/EwUnaryMat.h>
#include <runtime/local/kernels/Gemv.h>
#include <runtime/local/kernels/RandMatrix.h>
#include <runtime/local/kernels/Seq.h>
#include <runtime/local/kernels/Solve.h>
#include <runtime/local/kernels/Syrk.h>
#include <runtime/local/kernels/Transpose.h>

#include <cblas.h>

#include <cstdint>
#include <cstring>
#include <memory>
#include <stdexcept>

namespace {

// Non-owning DenseMatrix over caller memory (a view is taken when the leading dimension exceeds the column count).
template <typename VT> struct Wrapped {
    DenseMatrix<VT> *base = nullptr;
    DenseMatrix<VT> *m = nullptr;
    Wrapped(const VT *p, int64_t rows, int64_t cols, int64_t ld) {
        std::shared_ptr<VT[]> sp(const_cast<VT *>(p), [](VT *) {});
        if (ld == cols || rows <= 1) {
            base = DataObjectFactory::create<DenseMatrix<VT>>((size_t)rows, (size_t)cols, sp);
            m = base;
        } else {
            base = DataObjectFactory::create<DenseMatrix<VT>>((size_t)rows, (size_t)ld, sp);
            m = DataObjectFactory::create<DenseMatrix<VT>>(base, 0, rows, 0, cols);
        }
    }
    ~Wrapped() {
        if (m != base)
            DataObjectFactory::destroy(m);
        DataObjectFactory::destroy(base);
    }
};

template <typename VT> void copy_out(const DenseMatrix<VT> *src, VT *dst, int64_t dst_ld) {
    for (size_t r = 0; r < src->getNumRows(); r++)
        memcpy(dst + r * dst_ld, src->getValues() + r * src->getRowSkip(), src->getNumCols() * sizeof(VT));
}

template <typename F> int guarded(F &&f) {
    try {
        f();
        return 0;
    } catch (const std::domain_error &) {
        return 5;
    } catch (const std::exception &) {
        return 1;
    }
}

template <typename VT>
int ew_binary(int op, const VT *lhs, int64_t lr, int64_t lc, int64_t lld, const VT *rhs, int64_t rr, int64_t rc,
              int64_t rld, VT *res, int64_t res_ld) {
    return guarded([&] {
        Wrapped<VT> L(lhs, lr, lc, lld), R(rhs, rr, rc, rld);
        DenseMatrix<VT> *out = nullptr;
        ewBinaryMat<DenseMatrix<VT>, DenseMatrix<VT>, DenseMatrix<VT>>(static_cast<BinaryOpCode>(op), out, L.m, R.m,
                                                                        nullptr);
        copy_out(out, res, res_ld);
        DataObjectFactory::destroy(out);
    });
}
template <typename VT>
int ew_binary_sca(int op, const VT *lhs, int64_t rows, int64_t cols, int64_t ld, VT s, VT *res, int64_t res_ld) {
    return guarded([&] {
        Wrapped<VT> L(lhs, rows, cols, ld);
        DenseMatrix<VT> *out = nullptr;
        ewBinaryObjSca<DenseMatrix<VT>, DenseMatrix<VT>, VT>(static_cast<BinaryOpCode>(op), out, L.m, s, nullptr);
        copy_out(out, res, res_ld);
        DataObjectFactory::destroy(out);
    });
}
template <typename VT>
int ew_unary(int op, const VT *arg, int64_t rows, int64_t cols, int64_t ld, VT *res, int64_t res_ld) {
    return guarded([&] {
        Wrapped<VT> A(arg, rows, cols, ld);
        DenseMatrix<VT> *out = nullptr;
        ewUnaryMat<DenseMatrix<VT>, DenseMatrix<VT>>(static_cast<UnaryOpCode>(op), out, A.m, nullptr);
        copy_out(out, res, res_ld);
        DataObjectFactory::destroy(out);
    });
}
bool is_idx(int op) { return op == (int)AggOpCode::IDXMIN || op == (int)AggOpCode::IDXMAX; }

template <typename VT>
int agg_row(int op, const VT *arg, int64_t rows, int64_t cols, int64_t ld, VT *res, uint64_t *res_idx,
            int64_t res_ld) {
    return guarded([&] {
        Wrapped<VT> A(arg, rows, cols, ld);
        if (is_idx(op)) {
            DenseMatrix<size_t> *out = nullptr;
            aggRow<DenseMatrix<size_t>, DenseMatrix<VT>>(static_cast<AggOpCode>(op), out, A.m, nullptr);
            for (int64_t r = 0; r < rows; r++)
                res_idx[r * res_ld] = out->getValues()[r * out->getRowSkip()];
            DataObjectFactory::destroy(out);
        } else {
            DenseMatrix<VT> *out = nullptr;
            aggRow<DenseMatrix<VT>, DenseMatrix<VT>>(static_cast<AggOpCode>(op), out, A.m, nullptr);
            copy_out(out, res, res_ld);
            DataObjectFactory::destroy(out);
        }
    });
}
template <typename VT>
int agg_col(int op, const VT *arg, int64_t rows, int64_t cols, int64_t ld, VT *res, uint64_t *res_idx) {
    return guarded([&] {
        Wrapped<VT> A(arg, rows, cols, ld);
        if (is_idx(op)) {
            DenseMatrix<size_t> *out = nullptr;
            aggCol<DenseMatrix<size_t>, DenseMatrix<VT>>(static_cast<AggOpCode>(op), out, A.m, nullptr);
            for (int64_t c = 0; c < cols; c++)
                res_idx[c] = out->getValues()[c];
            DataObjectFactory::destroy(out);
        } else {
            DenseMatrix<VT> *out = nullptr;
            aggCol<DenseMatrix<VT>, DenseMatrix<VT>>(static_cast<AggOpCode>(op), out, A.m, nullptr);
            copy_out(out, res, cols);
            DataObjectFactory::destroy(out);
        }
    });
}
template <typename VT> int agg_all(int op, const VT *arg, int64_t rows, int64_t cols, int64_t ld, VT *res) {
    return guarded([&] {
        Wrapped<VT> A(arg, rows, cols, ld);
        *res = aggAll<VT, DenseMatrix<VT>>(static_cast<AggOpCode>(op), A.m, nullptr);
    });
}

// Non-owning CSRMatrix over caller arrays (size_t indices as in CSRMatrix.h:70-72).
template <typename VT> CSRMatrix<VT> *wrap_csr(const VT *vals, const uint64_t *cidx, const uint64_t *roff, int64_t rows,
                                               int64_t cols, int64_t nnz) {
    CSRMatrix<VT> *m = DataObjectFactory::create<CSRMatrix<VT>>((size_t)rows, (size_t)cols, (size_t)nnz, false);
    memcpy(m->getValues(), vals, sizeof(VT) * nnz);
    memcpy(m->getColIdxs(), cidx, sizeof(size_t) * nnz);
    memcpy(m->getRowOffsets(), roff, sizeof(size_t) * (rows + 1));
    return m;
}

} // namespace

#define DEF_TYPED(NAME, VT)                                                                                            \
    extern "C" int ref_ew_binary_##NAME(int op, const VT *lhs, int64_t lr, int64_t lc, int64_t lld, const VT *rhs,     \
                                        int64_t rr, int64_t rc, int64_t rld, VT *res, int64_t res_ld) {                \
        return ew_binary<VT>(op, lhs, lr, lc, lld, rhs, rr, rc, rld, res, res_ld);                                     \
    }                                                                                                                  \
    extern "C" int ref_ew_binary_sca_##NAME(int op, const VT *lhs, int64_t rows, int64_t cols, int64_t ld, VT s,       \
                                            VT *res, int64_t res_ld) {                                                 \
        return ew_binary_sca<VT>(op, lhs, rows, cols, ld, s, res, res_ld);                                             \
    }                                                                                                                  \
    extern "C" int ref_ew_unary_##NAME(int op, const VT *arg, int64_t rows, int64_t cols, int64_t ld, VT *res,         \
                                       int64_t res_ld) {                                                               \
        return ew_unary<VT>(op, arg, rows, cols, ld, res, res_ld);                                                     \
    }                                                                                                                  \
    extern "C" int ref_agg_row_##NAME(int op, const VT *arg, int64_t rows, int64_t cols, int64_t ld, VT *res,          \
                                      uint64_t *res_idx, int64_t res_ld) {                                             \
        return agg_row<VT>(op, arg, rows, cols, ld, res, res_idx, res_ld);                                             \
    }                                                                                                                  \
    extern "C" int ref_agg_col_##NAME(int op, const VT *arg, int64_t rows, int64_t cols, int64_t ld, VT *res,          \
                                      uint64_t *res_idx) {                                                             \
        return agg_col<VT>(op, arg, rows, cols, ld, res, res_idx);                                                     \
    }                                                                                                                  \
    extern "C" int ref_agg_all_##NAME(int op, const VT *arg, int64_t rows, int64_t cols, int64_t ld, VT *res) {        \
        return agg_all<VT>(op, arg, rows, cols, ld, res);                                                              \
    }
DEF_TYPED(f64, double)
DEF_TYPED(f32, float)
DEF_TYPED(i64, int64_t)
// the elementwise binary kernels are also instantiated for the other integer value types (kernels.json)
#define DEF_TYPED_BINARY(NAME, VT)                                                                                     \
    extern "C" int ref_ew_binary_##NAME(int op, const VT *lhs, int64_t lr, int64_t lc, int64_t lld, const VT *rhs,     \
                                        int64_t rr, int64_t rc, int64_t rld, VT *res, int64_t res_ld) {                \
        return ew_binary<VT>(op, lhs, lr, lc, lld, rhs, rr, rc, rld, res, res_ld);                                     \
    }                                                                                                                  \
    extern "C" int ref_ew_binary_sca_##NAME(int op, const VT *lhs, int64_t rows, int64_t cols, int64_t ld, VT s,       \
                                            VT *res, int64_t res_ld) {                                                 \
        return ew_binary_sca<VT>(op, lhs, rows, cols, ld, s, res, res_ld);                                             \
    }
DEF_TYPED_BINARY(u64, uint64_t)
DEF_TYPED_BINARY(i32, int32_t)
DEF_TYPED_BINARY(u32, uint32_t)

extern "C" void ref_set_blas_threads(int n) { scipy_openblas_set_num_threads(n); }

// Syrk<Dense<double>,Dense<double>> (Syrk.h:51-71): res is n x n with n = trans_left ? cols : rows
extern "C" int ref_syrk_f64(const double *arg, int64_t rows, int64_t cols, int64_t ld, int trans_left, double *res) {
    return guarded([&] {
        Wrapped<double> A(arg, rows, cols, ld);
        DenseMatrix<double> *out = nullptr;
        syrk<DenseMatrix<double>, DenseMatrix<double>>(out, A.m, trans_left != 0, nullptr);
        copy_out(out, res, (int64_t)out->getNumCols());
        DataObjectFactory::destroy(out);
    });
}
// Gemv<Dense,Dense,Dense> (Gemv.h:51-63): res = t(mat) %*% vec, cols x 1
extern "C" int ref_gemv_f64(const double *mat, int64_t rows, int64_t cols, int64_t ld, const double *vec,
                            double *res) {
    return guarded([&] {
        Wrapped<double> A(mat, rows, cols, ld), V(vec, rows, 1, 1);
        DenseMatrix<double> *out = nullptr;
        gemv<DenseMatrix<double>, DenseMatrix<double>, DenseMatrix<double>>(out, A.m, V.m, nullptr);
        copy_out(out, res, 1);
        DataObjectFactory::destroy(out);
    });
}
// MatMul<Dense,Dense,Dense> for double: kernels/MatMul.cpp needs Eigen for its integer paths and cannot be compiled
// here, so its f64 dispatch (MatMul.cpp:248-290: dot -> cblas_ddot, matrix-vector -> cblas_dgemv, else cblas_dgemm
// row-major with rowSkip as leading dimension) is issued directly on the same BLAS.
extern "C" int ref_matmul_f64(const double *a, int64_t ar, int64_t ac, int64_t lda, const double *b, int64_t br,
                              int64_t bc, int64_t ldb, int transa, int transb, double *res) {
    const int64_t m = transa ? ac : ar, k = transa ? ar : ac, k2 = transb ? bc : br, n = transb ? br : bc;
    if (k != k2)
        return 1;
    if (m == 1 && n == 1)
        res[0] = cblas_ddot((int)k, a, transa ? (int)lda : 1, b, transb ? 1 : (int)ldb);
    else if (n == 1 && !transb)
        cblas_dgemv(CblasRowMajor, transa ? CblasTrans : CblasNoTrans, (int)ar, (int)ac, 1.0, a, (int)lda, b,
                    (int)ldb, 0.0, res, 1);
    else
        cblas_dgemm(CblasRowMajor, transa ? CblasTrans : CblasNoTrans, transb ? CblasTrans : CblasNoTrans, (int)m,
                    (int)n, (int)k, 1.0, a, (int)lda, b, (int)ldb, 0.0, res, (int)n);
    return 0;
}
// Solve<Dense,Dense,Dense> (Solve.h:86-116)
extern "C" int ref_solve_f64(const double *a, int64_t n, const double *b, double *x) {
    return guarded([&] {
        Wrapped<double> A(a, n, n, n), B(b, n, 1, 1);
        DenseMatrix<double> *out = nullptr;
        solve<DenseMatrix<double>, DenseMatrix<double>, DenseMatrix<double>>(out, A.m, B.m, nullptr);
        copy_out(out, x, 1);
        DataObjectFactory::destroy(out);
    });
}
// Transpose<Dense,Dense> (Transpose.h:51-76)
extern "C" int ref_transpose_f64(const double *arg, int64_t rows, int64_t cols, int64_t ld, double *res) {
    return guarded([&] {
        Wrapped<double> A(arg, rows, cols, ld);
        DenseMatrix<double> *out = nullptr;
        transpose<DenseMatrix<double>, DenseMatrix<double>>(out, A.m, nullptr);
        copy_out(out, res, rows);
        DataObjectFactory::destroy(out);
    });
}
// CTable<Dense<double>,Dense<int64>,Dense<int64>,double> (CTable.h:55-106)
extern "C" int ref_ctable_f64(const int64_t *lhs, const int64_t *rhs, int64_t n, double weight, int64_t res_rows,
                              int64_t res_cols, double *res, int64_t *out_rows, int64_t *out_cols) {
    return guarded([&] {
        Wrapped<int64_t> L(lhs, n, 1, 1), R(rhs, n, 1, 1);
        DenseMatrix<double> *out = nullptr;
        ctable<DenseMatrix<double>, DenseMatrix<int64_t>, DenseMatrix<int64_t>, double>(out, L.m, R.m, weight,
                                                                                         res_rows, res_cols, nullptr);
        *out_rows = (int64_t)out->getNumRows();
        *out_cols = (int64_t)out->getNumCols();
        if (res)
            copy_out(out, res, (int64_t)out->getNumCols());
        DataObjectFactory::destroy(out);
    });
}
// RandMatrix<Dense<double>> (RandMatrix.h:82-161): the generator behind DaphneDSL rand(rows, cols, min, max, sparsity, seed)
extern "C" int ref_rand_f64(int64_t rows, int64_t cols, double lo, double hi, double sparsity, int64_t seed,
                            double *res) {
    return guarded([&] {
        DenseMatrix<double> *out = nullptr;
        randMatrix<DenseMatrix<double>, double>(out, (size_t)rows, (size_t)cols, lo, hi, sparsity, seed, nullptr);
        copy_out(out, res, cols);
        DataObjectFactory::destroy(out);
    });
}
// Seq<Dense<double>> (Seq.h)
extern "C" int ref_seq_f64(double start, double end, double inc, double *res, int64_t cap, int64_t *n) {
    return guarded([&] {
        DenseMatrix<double> *out = nullptr;
        seq<DenseMatrix<double>>(out, start, end, inc, nullptr);
        *n = (int64_t)out->getNumRows();
        if (res && *n <= cap)
            copy_out(out, res, 1);
        DataObjectFactory::destroy(out);
    });
}

// ---- CSR ----
// EwBinaryMat<CSR,CSR,Dense> MUL (EwBinaryMat.h:254-317).  Outputs are sized for nnz(lhs); *out_nnz is the count kept.
extern "C" int ref_csr_ewmul_dense_f64(const double *vals, const uint64_t *cidx, const uint64_t *roff, int64_t rows,
                                       int64_t cols, int64_t nnz, const double *rhs, int64_t rr, int64_t rc,
                                       double *ovals, uint64_t *ocidx, uint64_t *oroff, int64_t *out_nnz) {
    return guarded([&] {
        CSRMatrix<double> *G = wrap_csr<double>(vals, cidx, roff, rows, cols, nnz);
        Wrapped<double> R(rhs, rr, rc, rc);
        CSRMatrix<double> *out = nullptr;
        ewBinaryMat<CSRMatrix<double>, CSRMatrix<double>, DenseMatrix<double>>(BinaryOpCode::MUL, out, G, R.m, nullptr);
        const size_t *ro = out->getRowOffsets();
        *out_nnz = (int64_t)ro[rows];
        memcpy(oroff, ro, sizeof(size_t) * (rows + 1));
        memcpy(ovals, out->getValues(), sizeof(double) * ro[rows]);
        memcpy(ocidx, out->getColIdxs(), sizeof(size_t) * ro[rows]);
        DataObjectFactory::destroy(out);
        DataObjectFactory::destroy(G);
    });
}
// AggRow<Dense,CSR> (AggRow.h:178-238)
extern "C" int ref_csr_agg_row_f64(int op, const double *vals, const uint64_t *cidx, const uint64_t *roff, int64_t rows,
                                   int64_t cols, int64_t nnz, double *res) {
    return guarded([&] {
        CSRMatrix<double> *G = wrap_csr<double>(vals, cidx, roff, rows, cols, nnz);
        DenseMatrix<double> *out = nullptr;
        aggRow<DenseMatrix<double>, CSRMatrix<double>>(static_cast<AggOpCode>(op), out, G, nullptr);
        copy_out(out, res, 1);
        DataObjectFactory::destroy(out);
        DataObjectFactory::destroy(G);
    });
}
// Gemv<Dense,CSR,Dense> (Gemv.h:79-117): res = mat %*% vec (no transpose in the CSR specialisation)
extern "C" int ref_csr_gemv_f64(const double *vals, const uint64_t *cidx, const uint64_t *roff, int64_t rows,
                                int64_t cols, int64_t nnz, const double *vec, int64_t vcols, double *res) {
    return guarded([&] {
        CSRMatrix<double> *G = wrap_csr<double>(vals, cidx, roff, rows, cols, nnz);
        Wrapped<double> V(vec, cols, vcols, vcols);
        DenseMatrix<double> *out = nullptr;
        gemv<DenseMatrix<double>, CSRMatrix<double>, DenseMatrix<double>>(out, G, V.m, nullptr);
        copy_out(out, res, vcols);
        DataObjectFactory::destroy(out);
        DataObjectFactory::destroy(G);
    });
}

// ReadDaphne / WriteDaphne for DenseMatrix (src/runtime/local/io/ReadDaphne.h:58-100, WriteDaphne.h:62-80): the
// reference's own serializer writes / reads the .dbdf file
#include <runtime/local/io/ReadDaphne.h>
#include <runtime/local/io/WriteDaphne.h>
#define REF_DBDF(NAME, VT)                                                                                             \
    extern "C" int ref_write_dbdf_##NAME(const char *path, const VT *v, int64_t rows, int64_t cols) {                  \
        return guarded([&] {                                                                                           \
            auto *m = DataObjectFactory::create<DenseMatrix<VT>>((size_t)rows, (size_t)cols, false);                   \
            memcpy(m->getValues(), v, sizeof(VT) * rows * cols);                                                       \
            writeDaphne(m, path);                                                                                      \
            DataObjectFactory::destroy(m);                                                                             \
        });                                                                                                            \
    }                                                                                                                  \
    extern "C" int ref_read_dbdf_##NAME(const char *path, VT *out, int64_t cap, int64_t *rows, int64_t *cols) {        \
        return guarded([&] {                                                                                           \
            DenseMatrix<VT> *m = nullptr;                                                                              \
            readDaphne(m, path);                                                                                       \
            *rows = (int64_t)m->getNumRows();                                                                          \
            *cols = (int64_t)m->getNumCols();                                                                          \
            if (*rows * *cols <= cap)                                                                                  \
                memcpy(out, m->getValues(), sizeof(VT) * *rows * *cols);                                               \
            DataObjectFactory::destroy(m);                                                                             \
        });                                                                                                            \
    }
REF_DBDF(f64, double)
REF_DBDF(f32, float)
REF_DBDF(i64, int64_t)
