// Device plumbing of the native engine: error checks, owned device and pinned buffers, a bump arena
// for a step's activations (nothing is allocated inside a step), and the library matrix products
// (cuBLAS / cuBLASLt called directly, as the reference's engine calls cublasGemmEx,
// src/cuda/ops/matmul.cu:194-204).
#pragma once
#include <cublasLt.h>
#include <cublas_v2.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstdint>
#include <map>
#include <stdexcept>
#include <string>
#include <tuple>
#include <vector>

namespace easygpt::engine {

struct DeviceError : std::runtime_error {
    using std::runtime_error::runtime_error;
};

inline void cuda_check(cudaError_t e, const char* what) {
    if (e != cudaSuccess) throw DeviceError(std::string(what) + ": " + cudaGetErrorString(e));
}
#define EG_CUDA(call) ::easygpt::engine::cuda_check((call), #call)

// A kernel launcher of the kernel library returns the launch's cudaError_t as an int; 1 (invalid value) is also
// how a kernel refuses a size it does not take.
inline void launch_check(int code, const char* what) {
    if (code != 0)
        throw DeviceError(std::string(what) + ": CUDA error " + std::to_string(code) + (code == 1 ? " (a size this kernel does not take)" : "") +
                          " " + cudaGetErrorString((cudaError_t)code));
}

enum class DType { F32 = 0, BF16 = 1 };          // the kernel library's dtype codes
inline size_t dtype_size(DType t) { return t == DType::F32 ? 4 : 2; }

class DeviceBuffer {
public:
    DeviceBuffer() = default;
    explicit DeviceBuffer(size_t bytes, bool zero = false) { allocate(bytes, zero); }
    ~DeviceBuffer() { release(); }
    DeviceBuffer(const DeviceBuffer&) = delete;
    DeviceBuffer& operator=(const DeviceBuffer&) = delete;
    DeviceBuffer(DeviceBuffer&& o) noexcept : p_(o.p_), bytes_(o.bytes_) { o.p_ = nullptr; o.bytes_ = 0; }
    DeviceBuffer& operator=(DeviceBuffer&& o) noexcept {
        if (this != &o) { release(); p_ = o.p_; bytes_ = o.bytes_; o.p_ = nullptr; o.bytes_ = 0; }
        return *this;
    }
    void allocate(size_t bytes, bool zero = false) {
        release();
        bytes_ = bytes ? bytes : 16;
        cudaError_t e = cudaMalloc(&p_, bytes_);
        if (e != cudaSuccess) {
            p_ = nullptr;
            throw DeviceError("cannot allocate " + std::to_string(bytes_ >> 20) + " MiB of device memory: " + cudaGetErrorString(e));
        }
        if (zero) EG_CUDA(cudaMemset(p_, 0, bytes_));
    }
    void release() {
        if (p_) cudaFree(p_);
        p_ = nullptr;
        bytes_ = 0;
    }
    template <class T = void> T* as() const { return static_cast<T*>(p_); }
    void* get() const { return p_; }
    size_t bytes() const { return bytes_; }

private:
    void* p_ = nullptr;
    size_t bytes_ = 0;
};

class PinnedBuffer {
public:
    PinnedBuffer() = default;
    ~PinnedBuffer() { if (p_) cudaFreeHost(p_); }
    PinnedBuffer(const PinnedBuffer&) = delete;
    PinnedBuffer& operator=(const PinnedBuffer&) = delete;
    void ensure(size_t bytes) {
        if (bytes <= bytes_) return;
        if (p_) cudaFreeHost(p_);
        p_ = nullptr;
        size_t cap = 4096;
        while (cap < bytes) cap *= 2;
        EG_CUDA(cudaMallocHost(&p_, cap));
        bytes_ = cap;
    }
    template <class T> T* as() const { return static_cast<T*>(p_); }
    size_t bytes() const { return bytes_; }

private:
    void* p_ = nullptr;
    size_t bytes_ = 0;
};

// A step's activations: one block handed out front to back and taken back whole.  A captured step
// owns an arena of its own, so the addresses inside its graph stay valid.
class Arena {
public:
    explicit Arena(size_t bytes) : block_(bytes), used_(0) {}
    Arena(Arena&&) = default;
    void* take(size_t bytes) {
        const size_t at = (used_ + 255) & ~size_t(255);
        if (at + bytes > block_.bytes())
            throw DeviceError("a step needs more activation memory than its arena holds (" + std::to_string(block_.bytes() >> 20) +
                              " MiB); raise max_batch_tokens or lower the step's size");
        used_ = at + bytes;
        return block_.as<char>() + at;
    }
    template <class T> T* take_n(size_t n) { return static_cast<T*>(take(n * sizeof(T))); }
    void reset() { used_ = 0; }
    size_t used() const { return used_; }
    size_t capacity() const { return block_.bytes(); }

private:
    DeviceBuffer block_;
    size_t used_;
};

// The activation memory of one step: what lives for the whole step, and two arenas that the sub-layers use in turn.
struct ArenaSizes {
    size_t step = 0, sub = 0;
};
struct StepArenas {
    explicit StepArenas(const ArenaSizes& sizes) : sizes(sizes), step(sizes.step), sub{Arena(sizes.sub), Arena(sizes.sub)} {}
    bool holds(const ArenaSizes& need) const { return sizes.step >= need.step && sizes.sub >= need.sub; }
    void reset() {
        step.reset();
        sub[0].reset();
        sub[1].reset();
    }
    ArenaSizes sizes;
    Arena step;
    Arena sub[2];
};

// out[M,N] = x[M,K] w[N,K]^T (+ bias) through the library.  Row-major operands are handed over as their
// column-major transposes: out^T [N,M] = w (transposed read) times x^T.
class Blas {
public:
    Blas() {
        if (cublasCreate(&handle_) != CUBLAS_STATUS_SUCCESS) throw DeviceError("cublasCreate failed");
        if (cublasLtCreate(&lt_) != CUBLAS_STATUS_SUCCESS) throw DeviceError("cublasLtCreate failed");
        workspace_.allocate(kWorkspace);
        // a workspace of our own: the library then allocates nothing, also not while a stream is being captured
        cublasSetWorkspace(handle_, workspace_.get(), kWorkspace);
    }
    ~Blas() {
        for (auto& kv : plans_) {
            cublasLtMatmulDescDestroy(kv.second.desc);
            cublasLtMatrixLayoutDestroy(kv.second.a);
            cublasLtMatrixLayoutDestroy(kv.second.b);
            cublasLtMatrixLayoutDestroy(kv.second.c);
        }
        if (lt_) cublasLtDestroy(lt_);
        if (handle_) cublasDestroy(handle_);
    }
    Blas(const Blas&) = delete;
    Blas& operator=(const Blas&) = delete;

    // bfloat16 operands; out bfloat16 (bias, if any, bfloat16 and added in the product's epilogue) or float32 (no bias)
    void gemm_bf16(cudaStream_t stream, const void* x, long long ldx, const void* w, long long ldw, const void* bias_bf16, void* out,
                   long long ldo, int M, int N, int K, bool out_f32) {
        if (bias_bf16 == nullptr) {
            const float one = 1.0f, zero = 0.0f;
            cublasSetStream(handle_, stream);
            const cublasStatus_t st = cublasGemmEx(handle_, CUBLAS_OP_T, CUBLAS_OP_N, N, M, K, &one, w, CUDA_R_16BF, (int)ldw, x, CUDA_R_16BF,
                                                   (int)ldx, &zero, out, out_f32 ? CUDA_R_32F : CUDA_R_16BF, (int)ldo, CUBLAS_COMPUTE_32F,
                                                   CUBLAS_GEMM_DEFAULT);
            if (st != CUBLAS_STATUS_SUCCESS) throw DeviceError("cublasGemmEx failed with status " + std::to_string((int)st));
            return;
        }
        if (out_f32) throw DeviceError("a library product with bias writes bfloat16");
        Plan& plan = plan_for(M, N, K, ldx, ldw, ldo);
        const float one = 1.0f, zero = 0.0f;
        cublasLtMatmulDescSetAttribute(plan.desc, CUBLASLT_MATMUL_DESC_BIAS_POINTER, &bias_bf16, sizeof(bias_bf16));
        const cublasStatus_t st = cublasLtMatmul(lt_, plan.desc, &one, w, plan.a, x, plan.b, &zero, out, plan.c, out, plan.c, &plan.algo,
                                                 workspace_.get(), kWorkspace, stream);
        if (st != CUBLAS_STATUS_SUCCESS) throw DeviceError("cublasLtMatmul failed with status " + std::to_string((int)st));
    }

private:
    static constexpr size_t kWorkspace = 64u << 20;
    struct Plan {
        cublasLtMatmulDesc_t desc;
        cublasLtMatrixLayout_t a, b, c;
        cublasLtMatmulAlgo_t algo;
    };
    Plan& plan_for(int M, int N, int K, long long ldx, long long ldw, long long ldo) {
        const auto key = std::make_tuple(M, N, K, ldx, ldw, ldo);
        auto it = plans_.find(key);
        if (it != plans_.end()) return it->second;
        Plan p;
        auto ok = [](cublasStatus_t s, const char* what) {
            if (s != CUBLAS_STATUS_SUCCESS) throw DeviceError(std::string(what) + " failed with status " + std::to_string((int)s));
        };
        ok(cublasLtMatmulDescCreate(&p.desc, CUBLAS_COMPUTE_32F, CUDA_R_32F), "cublasLtMatmulDescCreate");
        const cublasOperation_t ta = CUBLAS_OP_T, tb = CUBLAS_OP_N;
        ok(cublasLtMatmulDescSetAttribute(p.desc, CUBLASLT_MATMUL_DESC_TRANSA, &ta, sizeof(ta)), "transa");
        ok(cublasLtMatmulDescSetAttribute(p.desc, CUBLASLT_MATMUL_DESC_TRANSB, &tb, sizeof(tb)), "transb");
        const cublasLtEpilogue_t epi = CUBLASLT_EPILOGUE_BIAS;
        ok(cublasLtMatmulDescSetAttribute(p.desc, CUBLASLT_MATMUL_DESC_EPILOGUE, &epi, sizeof(epi)), "epilogue");
        const cudaDataType_t bias_type = CUDA_R_16BF;
        ok(cublasLtMatmulDescSetAttribute(p.desc, CUBLASLT_MATMUL_DESC_BIAS_DATA_TYPE, &bias_type, sizeof(bias_type)), "bias type");
        ok(cublasLtMatrixLayoutCreate(&p.a, CUDA_R_16BF, K, N, ldw), "layout a");      // w as stored: K x N column-major, read transposed
        ok(cublasLtMatrixLayoutCreate(&p.b, CUDA_R_16BF, K, M, ldx), "layout b");
        ok(cublasLtMatrixLayoutCreate(&p.c, CUDA_R_16BF, N, M, ldo), "layout c");
        cublasLtMatmulPreference_t pref;
        ok(cublasLtMatmulPreferenceCreate(&pref), "preference");
        const size_t ws = kWorkspace;
        cublasLtMatmulPreferenceSetAttribute(pref, CUBLASLT_MATMUL_PREF_MAX_WORKSPACE_BYTES, &ws, sizeof(ws));
        cublasLtMatmulHeuristicResult_t found;
        int n = 0;
        const cublasStatus_t st = cublasLtMatmulAlgoGetHeuristic(lt_, p.desc, p.a, p.b, p.c, p.c, pref, 1, &found, &n);
        cublasLtMatmulPreferenceDestroy(pref);
        if (st != CUBLAS_STATUS_SUCCESS || n == 0) throw DeviceError("cuBLASLt has no algorithm for a product with bias of this shape");
        p.algo = found.algo;
        return plans_.emplace(key, p).first->second;
    }

    cublasHandle_t handle_ = nullptr;
    cublasLtHandle_t lt_ = nullptr;
    DeviceBuffer workspace_;
    std::map<std::tuple<int, int, int, long long, long long, long long>, Plan> plans_;
};

}  // namespace easygpt::engine
