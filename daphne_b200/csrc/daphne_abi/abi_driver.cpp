// TEST DRIVER for the adapter: plays the role of DAPHNE's JIT-compiled code.  It owns real DenseMatrix objects, looks
// the kernels up BY SYMBOL NAME in the adapter library (dlsym) and calls them with the (results..., args..., kId, ctx)
// convention of the generated wrappers (src/runtime/local/kernels/genKernelInst.py:183-262), then reads the results
// back through DenseMatrix::getValues() -- i.e. through the residency layer.
#include <B200Adapter.h>
#include <runtime/local/datastructures/CSRMatrix.h>

#include <dlfcn.h>

#include <cstring>

namespace {
DaphneContext g_ctx;
void *sym(const char *name) {
    void *p = dlsym(RTLD_DEFAULT, name);
    if (!p)
        throw std::runtime_error(std::string("symbol not found: ") + name);
    return p;
}
DenseMatrix<double> *host_matrix(const double *v, int64_t r, int64_t c) {
    auto *m = DataObjectFactory::create<DenseMatrix<double>>((size_t)r, (size_t)c, false);
    memcpy(m->getValues(), v, sizeof(double) * r * c);
    return m;
}
int copy_out(DenseMatrix<double> *m, double *out, int64_t cap, int64_t *r, int64_t *c) {
    *r = (int64_t)m->getNumRows();
    *c = (int64_t)m->getNumCols();
    if (*r * *c > cap)
        return 3;
    const double *v = static_cast<const DenseMatrix<double> *>(m)->getValues(); // device -> host through the MDO
    for (int64_t i = 0; i < *r; i++)
        memcpy(out + i * *c, v + i * m->getRowSkip(), sizeof(double) * *c);
    return 0;
}
char g_err[1024];
template <typename F> int guarded(F &&f) {
    try {
        return f();
    } catch (const std::exception &e) {
        snprintf(g_err, sizeof(g_err), "%s", e.what());
        return 1;
    }
}
} // namespace

extern "C" {
const char *drv_last_error() { return g_err; }

int drv_init() {
    return guarded([] {
        reinterpret_cast<void (*)(int, DaphneContext *)>(sym("CUDA_createCUDAContext"))(0, &g_ctx);
        return 0;
    });
}
// res = kernel(arg): aggRow / aggCol / transpose style
int drv_unary(const char *name, const double *a, int64_t ar, int64_t ac, double *out, int64_t cap, int64_t *r,
              int64_t *c) {
    return guarded([&] {
        auto *A = host_matrix(a, ar, ac);
        DenseMatrix<double> *R = nullptr;
        reinterpret_cast<void (*)(DenseMatrix<double> **, const DenseMatrix<double> *, int, DaphneContext *)>(
            sym(name))(&R, A, 1, &g_ctx);
        int rc = copy_out(R, out, cap, r, c);
        DataObjectFactory::destroy(A, R);
        return rc;
    });
}
// scalar = kernel(arg): aggAll style
int drv_scalar(const char *name, const double *a, int64_t ar, int64_t ac, double *out) {
    return guarded([&] {
        auto *A = host_matrix(a, ar, ac);
        reinterpret_cast<void (*)(double *, const DenseMatrix<double> *, int, DaphneContext *)>(sym(name))(out, A, 2,
                                                                                                      &g_ctx);
        DataObjectFactory::destroy(A);
        return 0;
    });
}
// res = kernel(lhs, rhs): ewBinaryMat / gemv / solve style
int drv_binary(const char *name, const double *a, int64_t ar, int64_t ac, const double *b, int64_t br, int64_t bc,
               double *out, int64_t cap, int64_t *r, int64_t *c) {
    return guarded([&] {
        auto *A = host_matrix(a, ar, ac);
        auto *B = host_matrix(b, br, bc);
        DenseMatrix<double> *R = nullptr;
        reinterpret_cast<void (*)(DenseMatrix<double> **, const DenseMatrix<double> *, const DenseMatrix<double> *,
                                  int, DaphneContext *)>(sym(name))(&R, A, B, 3, &g_ctx);
        int rc = copy_out(R, out, cap, r, c);
        DataObjectFactory::destroy(A, B, R);
        return rc;
    });
}
int drv_binary_sca(const char *name, const double *a, int64_t ar, int64_t ac, double s, double *out, int64_t cap,
                   int64_t *r, int64_t *c) {
    return guarded([&] {
        auto *A = host_matrix(a, ar, ac);
        DenseMatrix<double> *R = nullptr;
        reinterpret_cast<void (*)(DenseMatrix<double> **, const DenseMatrix<double> *, double, int, DaphneContext *)>(
            sym(name))(&R, A, s, 4, &g_ctx);
        int rc = copy_out(R, out, cap, r, c);
        DataObjectFactory::destroy(A, R);
        return rc;
    });
}
int drv_matmul(const double *a, int64_t ar, int64_t ac, const double *b, int64_t br, int64_t bc, int ta, int tb,
               double *out, int64_t cap, int64_t *r, int64_t *c) {
    return guarded([&] {
        auto *A = host_matrix(a, ar, ac);
        auto *B = host_matrix(b, br, bc);
        DenseMatrix<double> *R = nullptr;
        reinterpret_cast<void (*)(DenseMatrix<double> **, const DenseMatrix<double> *, const DenseMatrix<double> *,
                                  bool, bool, int, DaphneContext *)>(
            sym("CUDA_matMul__DenseMatrix_double__DenseMatrix_double__DenseMatrix_double__bool__bool"))(
            &R, A, B, ta != 0, tb != 0, 5, &g_ctx);
        int rc = copy_out(R, out, cap, r, c);
        DataObjectFactory::destroy(A, B, R);
        return rc;
    });
}
int drv_syrk(const double *a, int64_t ar, int64_t ac, int trans_left, double *out, int64_t cap, int64_t *r,
             int64_t *c) {
    return guarded([&] {
        auto *A = host_matrix(a, ar, ac);
        DenseMatrix<double> *R = nullptr;
        reinterpret_cast<void (*)(DenseMatrix<double> **, const DenseMatrix<double> *, bool, int, DaphneContext *)>(
            sym("CUDA_syrk__DenseMatrix_double__DenseMatrix_double__bool"))(&R, A, trans_left != 0, 6, &g_ctx);
        int rc = copy_out(R, out, cap, r, c);
        DataObjectFactory::destroy(A, R);
        return rc;
    });
}
// A chained call sequence whose intermediates never visit the host, including a row VIEW of a device-resident
// matrix: r = sumRow((X[r0:r1, ] - mu) * s) -- exercises handle passing, deferred chains and view offsets.
int drv_chain(const double *x, int64_t xr, int64_t xc, const double *mu, double s, int64_t r0, int64_t r1, double *out,
              int64_t cap, int64_t *r, int64_t *c) {
    return guarded([&] {
        using DM = DenseMatrix<double>;
        auto *X = host_matrix(x, xr, xc);
        auto *MU = host_matrix(mu, 1, xc);
        DM *X2 = nullptr, *D = nullptr, *S = nullptr, *R = nullptr;
        // X2 = X + 0 lives on the device only; the view below inherits its device placement
        reinterpret_cast<void (*)(DM **, const DM *, double, int, DaphneContext *)>(
            sym("CUDA_ewAdd__DenseMatrix_double__DenseMatrix_double__double"))(&X2, X, 0.0, 7, &g_ctx);
        auto *V = DataObjectFactory::create<DM>(X2, r0, r1);
        reinterpret_cast<void (*)(DM **, const DM *, const DM *, int, DaphneContext *)>(
            sym("CUDA_ewSub__DenseMatrix_double__DenseMatrix_double__DenseMatrix_double"))(&D, V, MU, 8, &g_ctx);
        reinterpret_cast<void (*)(DM **, const DM *, double, int, DaphneContext *)>(
            sym("CUDA_ewMul__DenseMatrix_double__DenseMatrix_double__double"))(&S, D, s, 9, &g_ctx);
        reinterpret_cast<void (*)(DM **, const DM *, int, DaphneContext *)>(
            sym("CUDA_sumRow__DenseMatrix_double__DenseMatrix_double"))(&R, S, 10, &g_ctx);
        int rc = copy_out(R, out, cap, r, c);
        DataObjectFactory::destroy(X, MU, X2, V, D, S, R);
        return rc;
    });
}
// The backend-"CPP" extension kernels (libB200ExtKernels.so), resolved by their catalog names: S = sqrt(X) stays on the
// device and feeds idxminRow (size_t result), meanCol and varCol; ctable builds a contingency matrix from int64
// coordinates.  out = [idxmin (xr) | mean (xc) | var (xc) | ctable (tr x tc)].
int drv_ext(const double *x, int64_t xr, int64_t xc, const int64_t *ys, const int64_t *xs, int64_t n, double weight,
            int64_t tr, int64_t tc, double *out) {
    return guarded([&] {
        using DM = DenseMatrix<double>;
        using DI = DenseMatrix<int64_t>;
        using DS = DenseMatrix<size_t>;
        auto *X = host_matrix(x, xr, xc);
        DM *S = nullptr, *M = nullptr, *V = nullptr, *T = nullptr;
        DS *I = nullptr;
        reinterpret_cast<void (*)(DM **, const DM *, int, DaphneContext *)>(
            sym("_ewSqrt__DenseMatrix_double__DenseMatrix_double"))(&S, X, 1, &g_ctx);
        reinterpret_cast<void (*)(DS **, const DM *, int, DaphneContext *)>(
            sym("_idxminRow__DenseMatrix_size_t__DenseMatrix_double"))(&I, S, 2, &g_ctx);
        reinterpret_cast<void (*)(DM **, const DM *, int, DaphneContext *)>(
            sym("_meanCol__DenseMatrix_double__DenseMatrix_double"))(&M, S, 3, &g_ctx);
        reinterpret_cast<void (*)(DM **, const DM *, int, DaphneContext *)>(
            sym("_varCol__DenseMatrix_double__DenseMatrix_double"))(&V, S, 4, &g_ctx);
        auto *Y = DataObjectFactory::create<DI>((size_t)n, 1, false);
        auto *Xs = DataObjectFactory::create<DI>((size_t)n, 1, false);
        memcpy(Y->getValues(), ys, sizeof(int64_t) * n);
        memcpy(Xs->getValues(), xs, sizeof(int64_t) * n);
        reinterpret_cast<void (*)(DM **, const DI *, const DI *, double, int64_t, int64_t, int, DaphneContext *)>(
            sym("_ctable__DenseMatrix_double__DenseMatrix_int64_t__DenseMatrix_int64_t__double__int64_t__int64_t"))(
            &T, Y, Xs, weight, tr, tc, 5, &g_ctx);
        const size_t *iv = static_cast<const DS *>(I)->getValues();
        for (int64_t r = 0; r < xr; r++)
            out[r] = (double)iv[r];
        int64_t rr, cc;
        copy_out(M, out + xr, xc, &rr, &cc);
        copy_out(V, out + xr + xc, xc, &rr, &cc);
        copy_out(T, out + xr + 2 * xc, tr * tc, &rr, &cc);
        DataObjectFactory::destroy(X, S, M, V, T, Y, Xs);
        DataObjectFactory::destroy(I);
        return 0;
    });
}
// A compiled pipeline body as the JIT would emit it (`_vect_cuda0`): calls kernels by their catalog names on its
// inputs (X: ROWS split, mu: broadcast row vector, s: scalar in the pointer slot), releases the inputs, returns
//   out0 = sumRow((X - mu) * s)    (ROWS)        out1 = sumCol(X - mu)    (ADD)
static void pipeline_body(DenseMatrix<double> ***outs, Structure **ins, DaphneContext *ctx) {
    using DM = DenseMatrix<double>;
    auto *X = static_cast<DM *>(ins[0]);
    auto *MU = static_cast<DM *>(ins[1]);
    double s;
    memcpy(&s, &ins[2], sizeof(double));
    DM *D = nullptr, *S = nullptr;
    reinterpret_cast<void (*)(DM **, const DM *, const DM *, int, DaphneContext *)>(
        sym("CUDA_ewSub__DenseMatrix_double__DenseMatrix_double__DenseMatrix_double"))(&D, X, MU, 1, ctx);
    reinterpret_cast<void (*)(DM **, const DM *, double, int, DaphneContext *)>(
        sym("CUDA_ewMul__DenseMatrix_double__DenseMatrix_double__double"))(&S, D, s, 2, ctx);
    reinterpret_cast<void (*)(DM **, const DM *, int, DaphneContext *)>(
        sym("CUDA_sumRow__DenseMatrix_double__DenseMatrix_double"))(outs[0], S, 3, ctx);
    reinterpret_cast<void (*)(DM **, const DM *, int, DaphneContext *)>(
        sym("CUDA_sumCol__DenseMatrix_double__DenseMatrix_double"))(outs[1], D, 4, ctx);
    DataObjectFactory::destroy(D, S, X, MU);
}
// calls the scheduler under DAPHNE's symbol name with that body; out = [out0 (xr) | out1 (xc)]
int drv_pipeline(const double *x, int64_t xr, int64_t xc, const double *mu, double s, double *out) {
    return guarded([&] {
        using DM = DenseMatrix<double>;
        auto *X = host_matrix(x, xr, xc);
        auto *MU = host_matrix(mu, 1, xc);
        Structure *inputs[3] = {X, MU, nullptr};
        memcpy(&inputs[2], &s, sizeof(double));
        bool is_scalar[3] = {false, false, true};
        int64_t splits[3] = {1, 0, 0}, combines[2] = {1, 3}, out_rows[2] = {xr, 1}, out_cols[2] = {1, xc};
        DM *outputs[2] = {nullptr, nullptr};
        void *funcs[1] = {reinterpret_cast<void *>(&pipeline_body)};
        reinterpret_cast<void (*)(DM **, size_t, bool *, Structure **, size_t, int64_t *, int64_t *, int64_t *, int64_t *,
                                  size_t, void **, int, DaphneContext *)>(
            sym("_vectorizedPipeline__DenseMatrix_double_variadic__size_t__bool__Structure_variadic__size_t__int64_t__"
                "int64_t__int64_t__int64_t__size_t__void_variadic"))(outputs, 2, is_scalar, inputs, 3, out_rows, out_cols,
                                                                     splits, combines, 1, funcs, 11, &g_ctx);
        int64_t r, c;
        int rc = copy_out(outputs[0], out, xr, &r, &c);
        if (rc == 0 && (r != xr || c != 1))
            rc = 4;
        if (rc == 0)
            rc = copy_out(outputs[1], out + xr, xc, &r, &c);
        DataObjectFactory::destroy(X, MU, outputs[0], outputs[1]);
        return rc;
    });
}

// A second compiled body with every kind of combine:
//   out0 = sumRow(X * s)  (ROWS)   out1 = sumCol(X) (ADD)   out2 = maxCol(X) (MAX)   out3 = minCol(X) (MIN)
//   out4 = t(maxRow(X))   (COLS)
static void pipeline_body_all(DenseMatrix<double> ***outs, Structure **ins, DaphneContext *ctx) {
    using DM = DenseMatrix<double>;
    auto *X = static_cast<DM *>(ins[0]);
    double s;
    memcpy(&s, &ins[1], sizeof(double));
    DM *S = nullptr, *M = nullptr;
    reinterpret_cast<void (*)(DM **, const DM *, double, int, DaphneContext *)>(
        sym("CUDA_ewMul__DenseMatrix_double__DenseMatrix_double__double"))(&S, X, s, 1, ctx);
    reinterpret_cast<void (*)(DM **, const DM *, int, DaphneContext *)>(
        sym("CUDA_sumRow__DenseMatrix_double__DenseMatrix_double"))(outs[0], S, 2, ctx);
    reinterpret_cast<void (*)(DM **, const DM *, int, DaphneContext *)>(
        sym("CUDA_sumCol__DenseMatrix_double__DenseMatrix_double"))(outs[1], X, 3, ctx);
    reinterpret_cast<void (*)(DM **, const DM *, int, DaphneContext *)>(
        sym("CUDA_maxCol__DenseMatrix_double__DenseMatrix_double"))(outs[2], X, 4, ctx);
    reinterpret_cast<void (*)(DM **, const DM *, int, DaphneContext *)>(
        sym("CUDA_minCol__DenseMatrix_double__DenseMatrix_double"))(outs[3], X, 5, ctx);
    reinterpret_cast<void (*)(DM **, const DM *, int, DaphneContext *)>(
        sym("CUDA_maxRow__DenseMatrix_double__DenseMatrix_double"))(&M, X, 6, ctx);
    reinterpret_cast<void (*)(DM **, const DM *, int, DaphneContext *)>(
        sym("CUDA_transpose__DenseMatrix_double__DenseMatrix_double"))(outs[4], M, 7, ctx);
    DataObjectFactory::destroy(S, M, X);
}
// out = [out0 (xr) | out1 (xc) | out2 (xc) | out3 (xc) | out4 (xr)]; x2 != 0: X is first replaced by X + 0 computed by a
// stand-alone kernel, so that the scheduler's input is device-resident (on the first device) and still deferred
int drv_pipeline_all(const double *x, int64_t xr, int64_t xc, double s, int x2, double *out) {
    return guarded([&] {
        using DM = DenseMatrix<double>;
        DM *X = host_matrix(x, xr, xc);
        if (x2) {
            DM *X2 = nullptr;
            reinterpret_cast<void (*)(DM **, const DM *, double, int, DaphneContext *)>(
                sym("CUDA_ewAdd__DenseMatrix_double__DenseMatrix_double__double"))(&X2, X, 0.0, 1, &g_ctx);
            DataObjectFactory::destroy(X);
            X = X2;
        }
        Structure *inputs[2] = {X, nullptr};
        memcpy(&inputs[1], &s, sizeof(double));
        bool is_scalar[2] = {false, true};
        int64_t splits[2] = {1, 0}, combines[5] = {1, 3, 5, 4, 2};
        int64_t out_rows[5] = {xr, 1, 1, 1, 1}, out_cols[5] = {1, xc, xc, xc, xr};
        DM *outputs[5] = {nullptr, nullptr, nullptr, nullptr, nullptr};
        void *funcs[1] = {reinterpret_cast<void *>(&pipeline_body_all)};
        reinterpret_cast<void (*)(DM **, size_t, bool *, Structure **, size_t, int64_t *, int64_t *, int64_t *, int64_t *,
                                  size_t, void **, int, DaphneContext *)>(
            sym("_vectorizedPipeline__DenseMatrix_double_variadic__size_t__bool__Structure_variadic__size_t__int64_t__"
                "int64_t__int64_t__int64_t__size_t__void_variadic"))(outputs, 5, is_scalar, inputs, 2, out_rows, out_cols,
                                                                     splits, combines, 1, funcs, 12, &g_ctx);
        const int64_t want_r[5] = {xr, 1, 1, 1, 1}, want_c[5] = {1, xc, xc, xc, xr};
        int64_t at = 0, r, c;
        int rc = 0;
        for (int o = 0; o < 5 && rc == 0; o++) {
            rc = copy_out(outputs[o], out + at, want_r[o] * want_c[o], &r, &c);
            if (rc == 0 && (r != want_r[o] || c != want_c[o]))
                rc = 4;
            at += want_r[o] * want_c[o];
        }
        DataObjectFactory::destroy(X, outputs[0], outputs[1], outputs[2], outputs[3], outputs[4]);
        return rc;
    });
}
// number of devices the scheduler spreads a pipeline over
int drv_devices() {
    int n = 0;
    db2_group_size(b200::group(&g_ctx), &n);
    return n;
}

// Connected components (test/api/cli/algorithms/components.daphne:14-26) as the kernel calls the script lowers to, by
// symbol name, on a real CSRMatrix:
//   c = seq(1, n); while (diff > 0 & iter <= maxi) { u = max(aggMax(G * t(c), 0), c); diff = sum(u != c); c = u; }
// G is given in the reference's layout (values, size_t column indices, size_t row offsets).  labels: n doubles.
int drv_components(const double *values, const uint64_t *col_idx, const uint64_t *row_off, int64_t n, int64_t maxi,
                   double *labels, int64_t *iterations) {
    return guarded([&] {
        using DM = DenseMatrix<double>;
        using CM = CSRMatrix<double>;
        const size_t nnz = (size_t)row_off[n];
        CM *G = DataObjectFactory::create<CM>((size_t)n, (size_t)n, nnz, false);
        memcpy(G->getValues(), values, nnz * sizeof(double));
        memcpy(G->getColIdxs(), col_idx, nnz * sizeof(size_t));
        memcpy(G->getRowOffsets(), row_off, (size_t)(n + 1) * sizeof(size_t));
        DM *c = DataObjectFactory::create<DM>((size_t)n, 1, false);
        for (int64_t i = 0; i < n; i++)
            c->getValues()[i] = (double)(i + 1);
        auto transpose = reinterpret_cast<void (*)(DM **, const DM *, int, DaphneContext *)>(
            sym("CUDA_transpose__DenseMatrix_double__DenseMatrix_double"));
        auto ew_mul = reinterpret_cast<void (*)(CM **, const CM *, const DM *, int, DaphneContext *)>(
            sym("_ewMul__CSRMatrix_double__CSRMatrix_double__DenseMatrix_double"));
        auto max_row = reinterpret_cast<void (*)(DM **, const CM *, int, DaphneContext *)>(
            sym("_maxRow__DenseMatrix_double__CSRMatrix_double"));
        auto ew_max = reinterpret_cast<void (*)(DM **, const DM *, const DM *, int, DaphneContext *)>(
            sym("CUDA_ewMax__DenseMatrix_double__DenseMatrix_double__DenseMatrix_double"));
        auto ew_neq = reinterpret_cast<void (*)(DM **, const DM *, const DM *, int, DaphneContext *)>(
            sym("CUDA_ewNeq__DenseMatrix_double__DenseMatrix_double__DenseMatrix_double"));
        auto sum_all = reinterpret_cast<void (*)(double *, const DM *, int, DaphneContext *)>(
            sym("CUDA_sumAll__double__DenseMatrix_double"));
        auto dec_ref = [](Structure *o) { DataObjectFactory::destroy(o); }; // what _decRef__Structure does
        double diff = 1.0;
        int64_t it = 1;
        while (diff > 0.0 && it <= maxi) {
            DM *tc = nullptr, *mx = nullptr, *u = nullptr, *ne = nullptr;
            CM *prod = nullptr;
            transpose(&tc, c, 1, &g_ctx);
            ew_mul(&prod, G, tc, 2, &g_ctx);
            max_row(&mx, prod, 3, &g_ctx);
            ew_max(&u, mx, c, 4, &g_ctx);
            ew_neq(&ne, u, c, 5, &g_ctx);
            sum_all(&diff, ne, 6, &g_ctx);
            dec_ref(tc);
            dec_ref(prod);
            dec_ref(mx);
            dec_ref(ne);
            dec_ref(c);
            c = u;
            it++;
        }
        *iterations = it - 1;
        int64_t r, cc;
        int rc = copy_out(c, labels, n, &r, &cc);
        dec_ref(c);
        dec_ref(G);
        return rc;
    });
}

} // extern "C"

namespace {
template <typename VT> DenseMatrix<VT> *host_matrix_t(const VT *v, int64_t r, int64_t c) {
    auto *m = DataObjectFactory::create<DenseMatrix<VT>>((size_t)r, (size_t)c, false);
    memcpy(m->getValues(), v, sizeof(VT) * r * c);
    return m;
}
template <typename VT> void copy_out_t(DenseMatrix<VT> *m, VT *out) {
    const VT *v = static_cast<const DenseMatrix<VT> *>(m)->getValues();
    for (size_t i = 0; i < m->getNumRows(); i++)
        memcpy(out + i * m->getNumCols(), v + i * m->getRowSkip(), sizeof(VT) * m->getNumCols());
}
// res = kernel(lhs, rhs) with matrices of value type VT; rhs == nullptr: res = kernel(lhs, scalar)
template <typename VT>
int binary_t(const char *name, const VT *a, int64_t ar, int64_t ac, const VT *b, int64_t br, int64_t bc, const VT *s,
             VT *out) {
    return guarded([&] {
        using DM = DenseMatrix<VT>;
        DM *A = host_matrix_t<VT>(a, ar, ac), *R = nullptr;
        if (b) {
            DM *B = host_matrix_t<VT>(b, br, bc);
            reinterpret_cast<void (*)(DM **, const DM *, const DM *, int, DaphneContext *)>(sym(name))(&R, A, B, 1, &g_ctx);
            DataObjectFactory::destroy(B);
        } else {
            reinterpret_cast<void (*)(DM **, const DM *, VT, int, DaphneContext *)>(sym(name))(&R, A, *s, 1, &g_ctx);
        }
        copy_out_t<VT>(R, out);
        DataObjectFactory::destroy(A, R);
        return 0;
    });
}
} // namespace

extern "C" {
// value type codes of include/daphne_b200.h; `out` holds ar * ac values
int drv_binary_typed(const char *name, int dtype, const void *a, int64_t ar, int64_t ac, const void *b, int64_t br,
                     int64_t bc, const void *scalar, void *out) {
    switch (dtype) {
    case DB2_F32: return binary_t<float>(name, (const float *)a, ar, ac, (const float *)b, br, bc, (const float *)scalar, (float *)out);
    case DB2_I64: return binary_t<int64_t>(name, (const int64_t *)a, ar, ac, (const int64_t *)b, br, bc, (const int64_t *)scalar, (int64_t *)out);
    case DB2_U64: return binary_t<uint64_t>(name, (const uint64_t *)a, ar, ac, (const uint64_t *)b, br, bc, (const uint64_t *)scalar, (uint64_t *)out);
    case DB2_I32: return binary_t<int32_t>(name, (const int32_t *)a, ar, ac, (const int32_t *)b, br, bc, (const int32_t *)scalar, (int32_t *)out);
    case DB2_U32: return binary_t<uint32_t>(name, (const uint32_t *)a, ar, ac, (const uint32_t *)b, br, bc, (const uint32_t *)scalar, (uint32_t *)out);
    default: return binary_t<double>(name, (const double *)a, ar, ac, (const double *)b, br, bc, (const double *)scalar, (double *)out);
    }
}
// res = matMul(lhs, rhs, transa, transb) by catalog name for an integer value type (DB2_I64 or DB2_I32); `out` holds
// the m x n result
int drv_matmul_int(const char *name, int dtype, const void *a, int64_t ar, int64_t ac, const void *b, int64_t br,
                   int64_t bc, int ta, int tb, void *out) {
    auto run = [&](auto zero) {
        using VT = decltype(zero);
        using DM = DenseMatrix<VT>;
        return guarded([&] {
            DM *A = host_matrix_t<VT>((const VT *)a, ar, ac), *B = host_matrix_t<VT>((const VT *)b, br, bc), *R = nullptr;
            reinterpret_cast<void (*)(DM **, const DM *, const DM *, bool, bool, int, DaphneContext *)>(sym(name))(
                &R, A, B, ta != 0, tb != 0, 1, &g_ctx);
            copy_out_t<VT>(R, (VT *)out);
            DataObjectFactory::destroy(A, B, R);
            return 0;
        });
    };
    return dtype == DB2_I32 ? run(int32_t{}) : run(int64_t{});
}
// fill through CUDA_fill__DenseMatrix_<vt>__<vt>__size_t__size_t for the one-byte value types (bool, uint8_t)
int drv_fill_u8(int as_bool, int value, int64_t rows, int64_t cols, uint8_t *out) {
    return guarded([&] {
        if (as_bool) {
            DenseMatrix<bool> *R = nullptr;
            reinterpret_cast<void (*)(DenseMatrix<bool> **, bool, size_t, size_t, int, DaphneContext *)>(
                sym("CUDA_fill__DenseMatrix_bool__bool__size_t__size_t"))(&R, value != 0, rows, cols, 1, &g_ctx);
            const bool *v = static_cast<const DenseMatrix<bool> *>(R)->getValues();
            for (int64_t i = 0; i < rows * cols; i++)
                out[i] = v[i] ? 1 : 0;
            DataObjectFactory::destroy(R);
        } else {
            DenseMatrix<uint8_t> *R = nullptr;
            reinterpret_cast<void (*)(DenseMatrix<uint8_t> **, uint8_t, size_t, size_t, int, DaphneContext *)>(
                sym("CUDA_fill__DenseMatrix_uint8_t__uint8_t__size_t__size_t"))(&R, (uint8_t)value, rows, cols, 1, &g_ctx);
            memcpy(out, static_cast<const DenseMatrix<uint8_t> *>(R)->getValues(), rows * cols);
            DataObjectFactory::destroy(R);
        }
        return 0;
    });
}
}
