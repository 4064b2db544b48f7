// GEMM entry points whose operands live in HOST memory, as every tensor of the reference does
// (src/tensor.zig:9-40: data is a host slice; src/cblas.zig:17-34 receives host pointers).
//
// A plain "copy in, multiply, copy out" sequence leaves the GPU idle for the whole transfer.  Here the
// product is cut into row panels of C: panel i's operand rows travel host->device on one copy stream
// while panel i-1 is multiplied on the compute stream and panel i-2's result travels device->host on a
// second copy stream (the two directions of the link are independent).  The device copies of the operands
// live in workspace slot 2 and keep the host layout (compacted leading dimensions).
#include <map>
#include <vector>

#include "common.cuh"

namespace znn {
namespace {

struct Pipe {
    cudaStream_t up = nullptr, down = nullptr;
    std::vector<cudaEvent_t> events;
    size_t used = 0;
};

thread_local std::map<int, Pipe> t_pipes;

Pipe* pipe()
{
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess) return nullptr;
    Pipe& p = t_pipes[dev];
    if (!p.up) {
        if (cudaStreamCreateWithFlags(&p.up, cudaStreamNonBlocking) != cudaSuccess) return nullptr;
        if (cudaStreamCreateWithFlags(&p.down, cudaStreamNonBlocking) != cudaSuccess) return nullptr;
    }
    p.used = 0;
    return &p;
}

cudaEvent_t next_event(Pipe* p)
{
    if (p->used == p->events.size()) {
        cudaEvent_t e = nullptr;
        if (cudaEventCreateWithFlags(&e, cudaEventDisableTiming) != cudaSuccess) return nullptr;
        p->events.push_back(e);
    }
    return p->events[p->used++];
}

// rows x width floats between a host matrix and its compact device copy
cudaError_t copy_block(float* dst, size_t dst_ld, const float* src, size_t src_ld, size_t rows, size_t width,
                       cudaMemcpyKind kind, cudaStream_t st)
{
    if (rows == 0 || width == 0) return cudaSuccess;
    if (dst_ld == width && src_ld == width) return cudaMemcpyAsync(dst, src, rows * width * sizeof(float), kind, st);
    return cudaMemcpy2DAsync(dst, dst_ld * sizeof(float), src, src_ld * sizeof(float), width * sizeof(float), rows, kind, st);
}

// record on `from`, make `to` wait
int chain(Pipe* p, cudaStream_t from, cudaStream_t to)
{
    cudaEvent_t e = next_event(p);
    if (!e) return fail(ZNN_ERR_CUDA, "could not create a CUDA event");
    ZNN_CUDA_OK(cudaEventRecord(e, from));
    ZNN_CUDA_OK(cudaStreamWaitEvent(to, e, 0));
    return ZNN_OK;
}

int panel_rows(int rows, int panels)
{
    if (panels <= 0) panels = rows >= 2048 ? (rows / 1024 > 16 ? 16 : rows / 1024) : 1;
    int pr = (rows + panels - 1) / panels;
    pr = (pr + 127) / 128 * 128;   // keeps every panel's first row on a tile boundary and 16-byte aligned
    return pr < 128 ? 128 : pr;
}

// Waits for everything the call queued; an error from the device surfaces here.
int drain(Pipe* p)
{
    ZNN_CUDA_OK(cudaStreamSynchronize(p->up));
    ZNN_CUDA_OK(cudaStreamSynchronize(stream()));
    ZNN_CUDA_OK(cudaStreamSynchronize(p->down));
    return ZNN_OK;
}

}  // namespace
}  // namespace znn

using namespace znn;

#define ZNN_TRY(expr)                    \
    do {                                 \
        int _rc = (expr);                \
        if (_rc != ZNN_OK) return _rc;   \
    } while (0)

extern "C" {

int znn_sgemm_host(int order, int trans_a, int trans_b, int M, int N, int K, float alpha, const float* A, int lda,
                   const float* B, int ldb, float beta, float* C, int ldc, int panels)
{
    ZNN_REQUIRE(order == ZNN_ROW_MAJOR, "only row-major (101) is supported, as in the reference");
    ZNN_REQUIRE(trans_a == ZNN_NO_TRANS || trans_a == ZNN_TRANS, "trans_a must be 111 or 112");
    ZNN_REQUIRE(trans_b == ZNN_NO_TRANS || trans_b == ZNN_TRANS, "trans_b must be 111 or 112");
    ZNN_REQUIRE(M >= 0 && N >= 0 && K >= 0, "negative dimension");
    if (M == 0 || N == 0) return ZNN_OK;
    ZNN_REQUIRE(C, "C is NULL");
    ZNN_REQUIRE(ldc >= N, "ldc (%d) < N (%d)", ldc, N);
    if (!stream()) return fail(ZNN_ERR_CUDA, "no CUDA device state; call znn_init (this library has no CPU fallback)");
    const bool mult = K > 0 && alpha != 0.0f;
    const bool an = trans_a == ZNN_NO_TRANS, bn = trans_b == ZNN_NO_TRANS;
    if (mult) {
        ZNN_REQUIRE(A && B, "A or B is NULL");
        ZNN_REQUIRE(lda >= (an ? K : M), "lda too small");
        ZNN_REQUIRE(ldb >= (bn ? N : K), "ldb too small");
    }
    Pipe* p = pipe();
    if (!p) return fail(ZNN_ERR_CUDA, "could not create the copy streams");

    const size_t na = mult ? (size_t)M * K : 0, nb = mult ? (size_t)K * N : 0, nc = (size_t)M * N;
    float* base = (float*)workspace_slot(2, (na + nb + nc) * sizeof(float) + 768);
    if (!base) return fail(ZNN_ERR_NOMEM, "could not reserve device copies of the operands");
    auto align64 = [](size_t n) { return (n + 63) / 64 * 64; };
    float* dA = base;
    float* dB = dA + align64(na);
    float* dC = dB + align64(nb);
    const int lda_d = an ? K : M, ldb_d = bn ? N : K;

    const int pr = panel_rows(M, panels);
    // whatever ran before on the compute stream may still use the device copies
    ZNN_TRY(chain(p, stream(), p->up));
    ZNN_TRY(chain(p, stream(), p->down));
    if (mult)
        ZNN_CUDA_OK(copy_block(dB, ldb_d, B, ldb, bn ? K : N, bn ? N : K, cudaMemcpyHostToDevice, p->up));

    for (int m0 = 0; m0 < M; m0 += pr) {
        const int mp = (M - m0 < pr) ? M - m0 : pr;
        if (mult) {
            if (an)
                ZNN_CUDA_OK(copy_block(dA + (size_t)m0 * K, K, A + (size_t)m0 * lda, lda, mp, K, cudaMemcpyHostToDevice, p->up));
            else
                ZNN_CUDA_OK(copy_block(dA + m0, M, A + m0, lda, K, mp, cudaMemcpyHostToDevice, p->up));
        }
        if (beta != 0.0f)
            ZNN_CUDA_OK(copy_block(dC + (size_t)m0 * N, N, C + (size_t)m0 * ldc, ldc, mp, N, cudaMemcpyHostToDevice, p->up));
        cudaStream_t cs = stream();
        ZNN_TRY(chain(p, p->up, cs));
        const float* a_panel = an ? dA + (size_t)m0 * K : dA + m0;
        ZNN_TRY(znn_sgemm(order, trans_a, trans_b, mp, N, K, alpha, a_panel, lda_d, dB, ldb_d, beta, dC + (size_t)m0 * N, N));
        ZNN_TRY(chain(p, cs, p->down));
        ZNN_CUDA_OK(copy_block(C + (size_t)m0 * ldc, ldc, dC + (size_t)m0 * N, N, mp, N, cudaMemcpyDeviceToHost, p->down));
    }
    return drain(p);
}

int znn_matmul_host_fwd_bwd(const float* A, const float* B, const float* dC, float* Cout, float* dA, float* dB,
                            int M, int K, int N, int accumulate, int panels)
{
    ZNN_REQUIRE(M > 0 && K > 0 && N > 0, "dimensions must be positive");
    ZNN_REQUIRE(A && B, "A or B is NULL");
    ZNN_REQUIRE(dC || (!dA && !dB), "gradients requested without dC");
    if (!stream()) return fail(ZNN_ERR_CUDA, "no CUDA device state; call znn_init (this library has no CPU fallback)");
    Pipe* p = pipe();
    if (!p) return fail(ZNN_ERR_CUDA, "could not create the copy streams");

    const size_t na = (size_t)M * K, nb = (size_t)K * N, nc = (size_t)M * N;
    auto align64 = [](size_t n) { return (n + 63) / 64 * 64; };
    const size_t total = 2 * align64(na) + 2 * align64(nb) + 2 * align64(nc);
    float* base = (float*)workspace_slot(2, total * sizeof(float));
    if (!base) return fail(ZNN_ERR_NOMEM, "could not reserve device copies of the operands");
    float* d_a = base;
    float* d_b = d_a + align64(na);
    float* d_dc = d_b + align64(nb);
    float* d_c = d_dc + align64(nc);
    float* d_da = d_c + align64(nc);
    float* d_db = d_da + align64(na);
    const float gbeta = accumulate ? 1.0f : 0.0f;

    const int pr = panel_rows(M, panels);
    const int pc = panel_rows(N, panels);
    ZNN_TRY(chain(p, stream(), p->up));
    ZNN_TRY(chain(p, stream(), p->down));

    // B first: every panel of C and of dA needs all of it.
    ZNN_CUDA_OK(cudaMemcpyAsync(d_b, B, nb * sizeof(float), cudaMemcpyHostToDevice, p->up));

    // C = A.B by row panels as A arrives (MatMul forward, src/autodiff.zig:107-133)
    for (int m0 = 0; m0 < M; m0 += pr) {
        const int mp = (M - m0 < pr) ? M - m0 : pr;
        ZNN_CUDA_OK(cudaMemcpyAsync(d_a + (size_t)m0 * K, A + (size_t)m0 * K, (size_t)mp * K * sizeof(float),
                                    cudaMemcpyHostToDevice, p->up));
        if (!Cout) continue;
        cudaStream_t cs = stream();
        ZNN_TRY(chain(p, p->up, cs));
        ZNN_TRY(znn_sgemm(ZNN_ROW_MAJOR, ZNN_NO_TRANS, ZNN_NO_TRANS, mp, N, K, 1.0f, d_a + (size_t)m0 * K, K, d_b, N, 0.0f,
                          d_c + (size_t)m0 * N, N));
        ZNN_TRY(chain(p, cs, p->down));
        ZNN_CUDA_OK(cudaMemcpyAsync(Cout + (size_t)m0 * N, d_c + (size_t)m0 * N, (size_t)mp * N * sizeof(float),
                                    cudaMemcpyDeviceToHost, p->down));
    }
    if (!dA && !dB) return drain(p);

    // dA (+)= dC.B^T by row panels as dC arrives (MatMul backward, src/autodiff.zig:593-641)
    for (int m0 = 0; m0 < M; m0 += pr) {
        const int mp = (M - m0 < pr) ? M - m0 : pr;
        ZNN_CUDA_OK(cudaMemcpyAsync(d_dc + (size_t)m0 * N, dC + (size_t)m0 * N, (size_t)mp * N * sizeof(float),
                                    cudaMemcpyHostToDevice, p->up));
        if (!dA) continue;
        if (accumulate)
            ZNN_CUDA_OK(cudaMemcpyAsync(d_da + (size_t)m0 * K, dA + (size_t)m0 * K, (size_t)mp * K * sizeof(float),
                                        cudaMemcpyHostToDevice, p->up));
        cudaStream_t cs = stream();
        ZNN_TRY(chain(p, p->up, cs));
        ZNN_TRY(znn_sgemm(ZNN_ROW_MAJOR, ZNN_NO_TRANS, ZNN_TRANS, mp, K, N, 1.0f, d_dc + (size_t)m0 * N, N, d_b, N, gbeta,
                          d_da + (size_t)m0 * K, K));
        ZNN_TRY(chain(p, cs, p->down));
        ZNN_CUDA_OK(cudaMemcpyAsync(dA + (size_t)m0 * K, d_da + (size_t)m0 * K, (size_t)mp * K * sizeof(float),
                                    cudaMemcpyDeviceToHost, p->down));
    }
    if (!dB) return drain(p);

    // dB (+)= A^T.dC needs every row of dC, so it is cut into column panels once dC is complete;
    // each finished panel leaves while the next one is multiplied.
    for (int n0 = 0; n0 < N; n0 += pc) {
        const int np = (N - n0 < pc) ? N - n0 : pc;
        if (accumulate) ZNN_CUDA_OK(copy_block(d_db + n0, N, dB + n0, N, K, np, cudaMemcpyHostToDevice, p->up));
        cudaStream_t cs = stream();
        ZNN_TRY(chain(p, p->up, cs));   // all of dC (queued above) has arrived
        ZNN_TRY(znn_sgemm(ZNN_ROW_MAJOR, ZNN_TRANS, ZNN_NO_TRANS, K, np, M, 1.0f, d_a, K, d_dc + n0, N, gbeta, d_db + n0, N));
        ZNN_TRY(chain(p, cs, p->down));
        ZNN_CUDA_OK(copy_block(dB + n0, N, d_db + n0, N, K, np, cudaMemcpyDeviceToHost, p->down));
    }
    return drain(p);
}

}  // extern "C"
