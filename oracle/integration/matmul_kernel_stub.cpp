// Test infrastructure, not product code: the replacement for the reference's src/matmul_kernel.cu that
// INTEGRATION.md shows, as a file that is really compiled. tests/test_integration_stub.py builds it against
// the reference's own src/tensor.h and this repository's include/akr_b200.h and checks that it defines every
// symbol src/bindings.cpp declares for this path (bindings.cpp:13-16, 142-143, 187-188, 260-261), so a change
// of either interface breaks the test. The block between the BEGIN / END markers is the text of INTEGRATION.md,
// section 2 (the same test compares them).
// BEGIN INTEGRATION SNIPPET
#include "tensor.h"
#include "akr_b200.h"

static akr_view as_view(const std::shared_ptr<Tensor>& t) {
    akr_view v{};
    v.data = t->data_ptr; v.ndim = (int32_t)t->shape.size(); v.dtype = (int32_t)t->dtype;   // DType and AKR_DTYPE_* agree
    for (size_t i = 0; i < t->shape.size(); ++i) { v.shape[i] = t->shape[i]; v.stride[i] = t->strides[i]; }
    return v;
}
static void check(int rc) {                      // same exception types the reference throws
    if (rc == AKR_OK) return;
    if (rc == AKR_ERR_INVALID) throw std::invalid_argument(akr_last_error());
    throw std::runtime_error(akr_last_error());
}

void set_tf32_enabled(bool e)        { akr_set_tf32(e); }          // matmul_kernel.cu:29-33
bool get_tf32_enabled()              { return akr_get_tf32() != 0; }
void set_cudnn_tf32_enabled(bool e)  { akr_set_cudnn_tf32(e); }    // :24-27, read by conv*_cudnn.cu
bool get_cudnn_tf32_enabled()        { return akr_get_cudnn_tf32() != 0; }
void cuda_synchronize()              { check(akr_synchronize()); } // :39-41

// forward, every dtype: the planner gives the broadcast result shape (same rules, same error texts)
static std::shared_ptr<Tensor> planned_output(const akr_view& va, const akr_view& vb, DType dt) {
    int64_t shape[AKR_MAX_DIMS]; int32_t nd = 0;
    check(akr_matmul_plan(&va, &vb, shape, &nd));
    return std::make_shared<Tensor>(std::vector<int>(shape, shape + nd), std::string("cuda"), dt);
}
std::shared_ptr<Tensor> run_cublas_matmul(std::shared_ptr<Tensor> a, std::shared_ptr<Tensor> b) {   // :111-143
    akr_view va = as_view(a), vb = as_view(b);
    auto out = planned_output(va, vb, DType::FLOAT32);
    akr_view vc = as_view(out);
    check(akr_matmul_fwd(&va, &vb, nullptr, &vc, AKR_MODE_GLOBAL, nullptr));   // no contiguity requirement
    return out;
}
std::shared_ptr<Tensor> run_cublas_matmul_a_bt(std::shared_ptr<Tensor> a, std::shared_ptr<Tensor> b) {  // :347-373
    auto out = std::make_shared<Tensor>(std::vector<int>{a->shape[0], b->shape[0]}, std::string("cuda"));
    akr_view va = as_view(a), vb = as_view(b), vc = as_view(out);
    check(akr_matmul_a_bt(&va, &vb, &vc, AKR_MODE_GLOBAL, nullptr));
    return out;
}
std::shared_ptr<Tensor> run_cublas_matmul_at_b(std::shared_ptr<Tensor> a, std::shared_ptr<Tensor> b) {  // :378-402
    auto out = std::make_shared<Tensor>(std::vector<int>{a->shape[1], b->shape[1]}, std::string("cuda"));
    akr_view va = as_view(a), vb = as_view(b), vc = as_view(out);
    check(akr_matmul_at_b(&va, &vb, &vc, AKR_MODE_GLOBAL, nullptr));
    return out;
}
static std::shared_ptr<Tensor> typed_forward(std::shared_ptr<Tensor> a, std::shared_ptr<Tensor> b) {  // :151-341
    akr_view va = as_view(a), vb = as_view(b);
    auto out = planned_output(va, vb, a->dtype);
    akr_view vc = as_view(out);
    check(akr_matmul_fwd_typed(&va, &vb, &vc, nullptr));   // float64 / int32 / int64, forward only
    return out;
}
std::shared_ptr<Tensor> run_cuda_matmul_f64(std::shared_ptr<Tensor> a, std::shared_ptr<Tensor> b) { return typed_forward(a, b); }
std::shared_ptr<Tensor> run_cuda_matmul_int_typed(std::shared_ptr<Tensor> a, std::shared_ptr<Tensor> b) { return typed_forward(a, b); }
// END INTEGRATION SNIPPET

// The reference's enum and the ABI's dtype codes must agree for the cast in as_view.
static_assert((int)DType::FLOAT32 == AKR_DTYPE_F32 && (int)DType::FLOAT64 == AKR_DTYPE_F64 &&
              (int)DType::INT32 == AKR_DTYPE_I32 && (int)DType::INT64 == AKR_DTYPE_I64, "dtype codes differ");
