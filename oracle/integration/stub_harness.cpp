// Test infrastructure, not product code: a C entry point around the drop-in stub (matmul_kernel_stub.cpp) so that
// a test can drive it from Python without the reference's binding layer. It builds the reference's OWN Tensor
// objects (src/tensor.h: CUDA constructor, CachingAllocator of src/allocator.h), fills them from host arrays, calls
// the three float32 entry points the reference's bindings call, and copies the result back.
#include "tensor.h"

#include <cuda_runtime.h>

#include <cstring>
#include <string>

std::shared_ptr<Tensor> run_cublas_matmul(std::shared_ptr<Tensor> a, std::shared_ptr<Tensor> b);
std::shared_ptr<Tensor> run_cublas_matmul_a_bt(std::shared_ptr<Tensor>, std::shared_ptr<Tensor>);
std::shared_ptr<Tensor> run_cublas_matmul_at_b(std::shared_ptr<Tensor>, std::shared_ptr<Tensor>);
void cuda_synchronize();
void set_tf32_enabled(bool enabled);

static std::shared_ptr<Tensor> upload(const float* host, const int* shape, int nd) {
    auto t = std::make_shared<Tensor>(std::vector<int>(shape, shape + nd), std::string("cuda"));
    cudaMemcpy(t->data_ptr, host, (size_t)t->size * sizeof(float), cudaMemcpyHostToDevice);
    return t;
}

// which: 0 run_cublas_matmul, 1 run_cublas_matmul_a_bt, 2 run_cublas_matmul_at_b; transpose_a: pass A as the
// reference's transposed VIEW (Tensor::transpose of the uploaded array), which the stock kernel refuses.
extern "C" int stub_run(int which, int tf32, int transpose_a, const float* a, const int* ashape, int and_,
                        const float* b, const int* bshape, int bnd, float* out, int out_capacity, int* oshape, int* ond,
                        char* err, int errlen) {
    try {
        set_tf32_enabled(tf32 != 0);
        auto A = upload(a, ashape, and_);
        auto B = upload(b, bshape, bnd);
        if (transpose_a) A = A->transpose(and_ - 2, and_ - 1);
        std::shared_ptr<Tensor> C = which == 0 ? run_cublas_matmul(A, B) : which == 1 ? run_cublas_matmul_a_bt(A, B)
                                                                                      : run_cublas_matmul_at_b(A, B);
        cuda_synchronize();
        if (C->size > out_capacity) throw std::runtime_error("output buffer too small");
        *ond = (int)C->shape.size();
        for (int i = 0; i < *ond; ++i) oshape[i] = C->shape[i];
        cudaMemcpy(out, C->data_ptr, (size_t)C->size * sizeof(float), cudaMemcpyDeviceToHost);
        set_tf32_enabled(false);
        return 0;
    } catch (const std::invalid_argument& e) {
        std::strncpy(err, e.what(), errlen - 1);
        return 1;
    } catch (const std::exception& e) {
        std::strncpy(err, e.what(), errlen - 1);
        return 2;
    }
}
