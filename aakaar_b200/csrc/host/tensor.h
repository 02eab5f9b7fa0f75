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

class Tensor : public std::enable_shared_from_this<Tensor> {
public:
    float* data = nullptr;
    int64_t size = 0;
    std::vector<int64_t> shape;
    std::vector<int64_t> strides;  // elements
    std::string device;            // "cuda" or "cpu" (host staging only)

    bool requires_grad = false;
    TensorPtr grad;
    std::shared_ptr<Node> grad_fn;
    TensorPtr base;  // parent of a view

    // Fresh contiguous allocation.
    Tensor(std::vector<int64_t> shp, const std::string& dev) : shape(std::move(shp)), device(dev) {
        size = 1;
        for (int64_t d : shape) {
            if (d <= 0) throw std::invalid_argument("Tensor dimensions must be positive");
            size *= d;
        }
        if (shape.size() > AKR_MAX_DIMS) throw std::invalid_argument("Tensors with more than 8 dimensions are not supported");
        strides = contiguous_strides(shape);
        if (device == "cuda") {
            check(akr_alloc((size_t)size, &owned_));
        } else if (device == "cpu") {
            owned_ = static_cast<float*>(::operator new((size_t)size * sizeof(float)));
        } else {
            throw std::invalid_argument("Unknown device '" + device + "' (expected 'cuda' or 'cpu')");
        }
        data = owned_;
    }

    // View of `parent` at element offset `off`.
    Tensor(const TensorPtr& parent, int64_t off, std::vector<int64_t> shp, std::vector<int64_t> strd)
        : shape(std::move(shp)), strides(std::move(strd)), device(parent->device),
          base(parent->base ? parent->base : parent) {
        size = 1;
        for (int64_t d : shape) size *= d;
        data = parent->data + off;
    }

    ~Tensor() {
        if (!base && owned_) {
            if (device == "cuda") akr_free(owned_, (size_t)size);
            else ::operator delete(owned_);
        }
    }
    Tensor(const Tensor&) = delete;
    Tensor& operator=(const Tensor&) = delete;

    bool is_contiguous() const { return strides == contiguous_strides(shape); }

    akr_view view() const {
        akr_view v;
        v.data = data;
        v.ndim = (int32_t)shape.size();
        v.dtype = AKR_DTYPE_F32;
        for (int i = 0; i < AKR_MAX_DIMS; ++i) {
            v.shape[i] = i < (int)shape.size() ? shape[i] : 1;
            v.stride[i] = i < (int)shape.size() ? strides[i] : 0;
        }
        return v;
    }

private:
    float* owned_ = nullptr;
};

inline void require_cuda(const TensorPtr& t, const char* op) {
    if (t->device != "cuda")
        throw std::runtime_error(std::string(op) +
                                 ": this build computes on CUDA (sm_100a) only; move the tensor with "
                                 ".to('cuda'). There is no CPU fallback.");
}

}  // namespace akrhost
