// Host-side tensor and autograd graph of the Python-facing module.
//
// Mirrors the part of the reference's Tensor / Node (src/tensor.h:37-58, 110-135, 239-260) that the
// matmul path touches: element strides, views that share their parent's buffer and keep it alive,
// device memory taken from the exact-size caching allocator behind the C ABI. All compute goes
// through include/akr_b200.h; there is no CPU arithmetic here.
#pragma once
#include <cstdint>
#include <functional>
#include <memory>
#include <stdexcept>
#include <string>
#include <vector>

#include "../../../include/akr_b200.h"

namespace akrhost {

class Tensor;
using TensorPtr = std::shared_ptr<Tensor>;

struct Node {
    std::function<std::vector<TensorPtr>(TensorPtr)> backward_fn;
    // Set by matmul / linear nodes only: the same backward, except that input 0 is known to be the
    // output of a tanh node and entry 0 of the result is the gradient with respect to THAT node's
    // input (the tanh' factor is applied in the epilogue of the dA product).
    std::function<std::vector<TensorPtr>(TensorPtr)> backward_through_tanh;
    std::vector<TensorPtr> inputs;
    std::string op_name;
    bool freed = false;
};

// Turns a C-ABI status into the exception type the reference throws for that class of error.
inline void check(int rc) {
    if (rc == AKR_OK) return;
    const std::string msg = akr_last_error();
    if (rc == AKR_ERR_INVALID) throw std::invalid_argument(msg);
    throw std::runtime_error(msg);
}

inline std::vector<int64_t> contiguous_strides(const std::vector<int64_t>& shape) {
    std::vector<int64_t> st(shape.size());
    int64_t acc = 1;
    for (int i = (int)shape.size() - 1; i >= 0; --i) {
        st[i] = acc;
        acc *= shape[i];
    }
    return st;
}

inline size_t dtype_size(int dtype) { return (dtype == AKR_DTYPE_F64 || dtype == AKR_DTYPE_I64) ? 8 : 4; }
inline const char* dtype_name(int dtype) {
    switch (dtype) {
        case AKR_DTYPE_F64: return "float64";
        case AKR_DTYPE_I32: return "int32";
        case AKR_DTYPE_I64: return "int64";
        default: return "float32";
    }
}

class Tensor : public std::enable_shared_from_this<Tensor> {
public:
    float* data = nullptr;         // first element; reinterpret according to `dtype`
    int dtype = AKR_DTYPE_F32;     // float32 everywhere except forward-only typed matmul
    int64_t size = 0;
    std::vector<int64_t> shape;
    std::vector<int64_t> strides;  // elements
    std::string device;            // "cuda" or "cpu" (host staging only)

    bool requires_grad = false;
    TensorPtr grad;
    std::shared_ptr<Node> grad_fn;
    TensorPtr base;  // parent of a view
    // Column sums of this tensor over all its leading dims (shape [last dim]), attached by the kernel that wrote
    // it when the consumer is known to want them: a gradient that flows into a Linear layer's output carries
    // that layer's bias gradient, so no extra pass over the gradient is needed.
    TensorPtr colsum;

    // Fresh contiguous allocation.
    Tensor(std::vector<int64_t> shp, const std::string& dev, int dt = AKR_DTYPE_F32)
        : dtype(dt), shape(std::move(shp)), device(dev) {
        size = 1;
        for (int64_t d : shape) {
            if (d <= 0) throw std::invalid_argument("Tensor dimensions must be positive");
            size *= d;
        }
        if (shape.size() > AKR_MAX_DIMS) throw std::invalid_argument("Tensors with more than 8 dimensions are not supported");
        strides = contiguous_strides(shape);
        if (device == "cuda") {
            check(akr_alloc(alloc_floats(), &owned_));   // the allocator counts in 4-byte units
        } else if (device == "cpu") {
            owned_ = static_cast<float*>(::operator new(nbytes()));
        } else {
            throw std::invalid_argument("Unknown device '" + device + "' (expected 'cuda' or 'cpu')");
        }
        data = owned_;
    }

    // View of `parent` at element offset `off`.
    Tensor(const TensorPtr& parent, int64_t off, std::vector<int64_t> shp, std::vector<int64_t> strd)
        : dtype(parent->dtype), shape(std::move(shp)), strides(std::move(strd)), device(parent->device),
          base(parent->base ? parent->base : parent) {
        size = 1;
        for (int64_t d : shape) size *= d;
        data = reinterpret_cast<float*>(reinterpret_cast<char*>(parent->data) + (size_t)off * dtype_size(dtype));
    }

    ~Tensor() {
        if (!base && owned_) {
            if (device == "cuda") akr_free(owned_, alloc_floats());
            else ::operator delete(owned_);
        }
    }
    Tensor(const Tensor&) = delete;
    Tensor& operator=(const Tensor&) = delete;

    bool is_contiguous() const { return strides == contiguous_strides(shape); }
    size_t nbytes() const { return (size_t)size * dtype_size(dtype); }
    size_t alloc_floats() const { return (nbytes() + 3) / 4; }

    akr_view view() const {
        akr_view v;
        v.data = data;
        v.ndim = (int32_t)shape.size();
        v.dtype = dtype;
        for (int i = 0; i < AKR_MAX_DIMS; ++i) {
            v.shape[i] = i < (int)shape.size() ? shape[i] : 1;
            v.stride[i] = i < (int)shape.size() ? strides[i] : 0;
        }
        return v;
    }

private:
    float* owned_ = nullptr;
};

inline void require_f32(const TensorPtr& t, const char* op) {
    if (t->dtype != AKR_DTYPE_F32)
        throw std::runtime_error(std::string(op) + ": only float32 is supported here (tensor is " +
                                 dtype_name(t->dtype) + "); the other dtypes support forward matmul only");
}

inline void require_cuda(const TensorPtr& t, const char* op) {
    if (t->device != "cuda")
        throw std::runtime_error(std::string(op) +
                                 ": this build computes on CUDA (sm_100a) only; move the tensor with "
                                 ".to('cuda'). There is no CPU fallback.");
}

}  // namespace akrhost
