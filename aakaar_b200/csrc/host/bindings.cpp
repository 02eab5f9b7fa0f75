// pybind11 module `_C` of aakaar_b200: the Python-facing surface of the matmul path, with the
// names and behaviour of the reference's module (src/bindings.cpp:2472-2874) for this path:
// Tensor (views, autograd, backward), cuda_matmul / __matmul__, from_numpy, set_tf32 switches,
// synchronize, the caching-allocator hooks, plus the few support ops the Linear training step
// needs. Every computation is a call into the C ABI of include/akr_b200.h; nothing here touches
// CUDA or PyTorch directly.
#include <pybind11/numpy.h>
#include <cmath>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include <algorithm>
#include <cstring>
#include <sstream>
#include <unordered_map>
#include <unordered_set>

#include "tensor.h"

namespace py = pybind11;
using namespace akrhost;

namespace {

bool g_grad_enabled = true;
// The all-ones gradient tensor_backward creates for a scalar root (null otherwise): a node that sees it knows
// its incoming gradient is exactly 1 without reading device memory.
const void* g_unit_root_grad = nullptr;

enum class DTypeEnum : int { float32 = AKR_DTYPE_F32, float64 = AKR_DTYPE_F64, int32 = AKR_DTYPE_I32, int64 = AKR_DTYPE_I64 };

TensorPtr make_cuda(const std::vector<int64_t>& shape) { return std::make_shared<Tensor>(shape, "cuda"); }

bool needs_graph(const TensorPtr& a) { return g_grad_enabled && a->requires_grad; }
bool needs_graph(const TensorPtr& a, const TensorPtr& b) {
    return g_grad_enabled && (a->requires_grad || b->requires_grad);
}

void attach(const TensorPtr& out, const char* name, std::vector<TensorPtr> inputs,
            std::function<std::vector<TensorPtr>(TensorPtr)> fn) {
    out->requires_grad = true;
    auto node = std::make_shared<Node>();
    node->inputs = std::move(inputs);
    node->op_name = name;
    node->backward_fn = std::move(fn);
    out->grad_fn = node;
}

// ------------------------------------------------------------------ basic ops

TensorPtr op_contiguous(const TensorPtr& t);

TensorPtr op_add_raw(const TensorPtr& a, const TensorPtr& b, bool multiply = false) {
    require_cuda(a, "add");
    require_f32(a, "add");
    require_cuda(b, "add");
    require_f32(b, "add");
    const size_t nd = std::max(a->shape.size(), b->shape.size());
    std::vector<int64_t> shape(nd);
    for (size_t i = 0; i < nd; ++i) {
        const int ia = (int)i - (int)(nd - a->shape.size()), ib = (int)i - (int)(nd - b->shape.size());
        const int64_t da = ia >= 0 ? a->shape[ia] : 1, db = ib >= 0 ? b->shape[ib] : 1;
        if (da != db && da != 1 && db != 1) throw std::invalid_argument("Shapes are not broadcastable");
        shape[i] = std::max(da, db);
    }
    auto out = make_cuda(shape);
    akr_view va = a->view(), vb = b->view(), vo = out->view();
    check((multiply ? akr_mul : akr_add)(&va, &vb, &vo, nullptr));
    return out;
}

// reduce_grad_to_shape of the reference (src/bindings.cpp:1467-1503) in one reduction launch.
TensorPtr op_sum_to(const TensorPtr& g, const std::vector<int64_t>& target) {
    if (g->shape == target) return g;
    auto out = make_cuda(target);
    akr_view vg = g->view(), vo = out->view();
    check(akr_sum_to(&vg, &vo, nullptr));
    return out;
}

TensorPtr op_scale(const TensorPtr& a, float s);

TensorPtr op_add(const TensorPtr& a, const TensorPtr& b) {
    auto out = op_add_raw(a, b);
    if (needs_graph(a, b)) {
        const auto sa = a->shape, sb = b->shape;
        attach(out, "add", {a, b}, [sa, sb](TensorPtr g) {
            return std::vector<TensorPtr>{op_sum_to(g, sa), op_sum_to(g, sb)};
        });
    }
    return out;
}

// Elementwise product with broadcasting; gradients g * b and g * a, each summed back to its operand's shape.
TensorPtr op_mul(const TensorPtr& a, const TensorPtr& b) {
    auto out = op_add_raw(a, b, true);
    if (needs_graph(a, b)) {
        attach(out, "mul", {a, b}, [a, b](TensorPtr g) {
            TensorPtr ga, gb;
            if (a->requires_grad) ga = op_sum_to(op_add_raw(g, b, true), a->shape);
            if (b->requires_grad) gb = op_sum_to(op_add_raw(g, a, true), b->shape);
            return std::vector<TensorPtr>{ga, gb};
        });
    }
    return out;
}

TensorPtr op_scale(const TensorPtr& a, float s) {
    require_cuda(a, "mul");
    require_f32(a, "mul");
    auto src = a->is_contiguous() ? a : op_contiguous(a);
    auto out = make_cuda(a->shape);
    check(akr_scale(src->data, s, out->data, (size_t)a->size, nullptr));
    if (needs_graph(a)) {
        attach(out, "mul_scalar", {a}, [s](TensorPtr g) {
            bool prev = g_grad_enabled;
            g_grad_enabled = false;
            auto r = op_scale(g, s);
            g_grad_enabled = prev;
            return std::vector<TensorPtr>{r};
        });
    }
    return out;
}

TensorPtr op_sub(const TensorPtr& a, const TensorPtr& b) { return op_add(a, op_scale(b, -1.0f)); }

TensorPtr scalar_tensor(float v) {
    auto t = make_cuda({1});
    check(akr_fill(t->data, v, 1, nullptr));
    return t;
}

TensorPtr op_contiguous(const TensorPtr& t) {
    if (t->is_contiguous()) return t;
    require_cuda(t, "contiguous");
    require_f32(t, "contiguous");
    auto out = make_cuda(t->shape);
    akr_view v = t->view();
    check(akr_contiguous(&v, out->data, nullptr));
    if (needs_graph(t)) {
        attach(out, "contiguous", {t}, [](TensorPtr g) { return std::vector<TensorPtr>{g}; });
    }
    return out;
}

TensorPtr op_transpose(const TensorPtr& t, int d0, int d1) {
    const int nd = (int)t->shape.size();
    if (d0 < 0) d0 += nd;
    if (d1 < 0) d1 += nd;
    if (d0 < 0 || d1 < 0 || d0 >= nd || d1 >= nd) throw std::out_of_range("transpose: dimension out of range");
    auto shape = t->shape;
    auto strides = t->strides;
    std::swap(shape[d0], shape[d1]);
    std::swap(strides[d0], strides[d1]);
    auto out = std::make_shared<Tensor>(t, 0, shape, strides);
    if (needs_graph(t)) {
        attach(out, "transpose", {t}, [d0, d1](TensorPtr g) {
            bool prev = g_grad_enabled;
            g_grad_enabled = false;
            auto r = op_transpose(g, d0, d1);
            g_grad_enabled = prev;
            return std::vector<TensorPtr>{r};
        });
    }
    return out;
}

TensorPtr op_view(const TensorPtr& t, std::vector<int64_t> new_shape, bool allow_copy) {
    int64_t known = 1;
    int infer = -1;
    for (size_t i = 0; i < new_shape.size(); ++i) {
        if (new_shape[i] == -1) {
            if (infer >= 0) throw std::invalid_argument("view: only one dimension can be inferred");
            infer = (int)i;
        } else {
            known *= new_shape[i];
        }
    }
    if (infer >= 0) {
        if (known == 0 || t->size % known != 0) throw std::invalid_argument("view: shape is invalid for input size");
        new_shape[infer] = t->size / known;
        known *= new_shape[infer];
    }
    if (known != t->size) throw std::invalid_argument("view: shape is invalid for input size");
    TensorPtr src = t;
    if (!t->is_contiguous()) {
        if (!allow_copy) throw std::invalid_argument("view requires a contiguous tensor. Call .contiguous() first.");
        src = op_contiguous(t);
    }
    auto out = std::make_shared<Tensor>(src, 0, new_shape, contiguous_strides(new_shape));
    if (needs_graph(src)) {
        const auto old_shape = src->shape;
        attach(out, "view", {src}, [old_shape](TensorPtr g) {
            bool prev = g_grad_enabled;
            g_grad_enabled = false;
            auto r = op_view(g, old_shape, true);
            g_grad_enabled = prev;
            return std::vector<TensorPtr>{r};
        });
    }
    return out;
}

TensorPtr op_tanh(const TensorPtr& t) {
    require_cuda(t, "tanh");
    require_f32(t, "tanh");
    auto src = op_contiguous(t);
    auto out = make_cuda(t->shape);
    check(akr_tanh_fwd(src->data, out->data, (size_t)t->size, nullptr));
    if (needs_graph(t)) {
        // The node is owned by `out`, so it refers to it weakly (no ownership cycle); whoever
        // runs backward through this node holds `out` alive.
        std::weak_ptr<Tensor> wout = out;
        attach(out, "tanh", {t}, [wout](TensorPtr g) {
            TensorPtr saved = wout.lock();
            if (!saved) throw std::runtime_error("tanh backward: forward output was released");
            auto gc = g->is_contiguous() ? g : op_contiguous(g);
            auto dx = make_cuda(saved->shape);
            check(akr_tanh_bwd(gc->data, saved->data, dx->data, (size_t)saved->size, nullptr));
            return std::vector<TensorPtr>{dx};
        });
    }
    return out;
}

TensorPtr op_sum_all(const TensorPtr& t) {
    require_cuda(t, "sum");
    require_f32(t, "sum");
    auto out = make_cuda({1});
    akr_view vg = t->view(), vo = out->view();
    check(akr_sum_to(&vg, &vo, nullptr));
    if (needs_graph(t)) {
        const auto shape = t->shape;
        attach(out, "sum", {t}, [shape](TensorPtr g) {
            // broadcast the scalar gradient: zeros(shape) + g
            auto z = make_cuda(shape);
            int64_t n = 1;
            for (auto d : shape) n *= d;
            check(akr_fill(z->data, 0.0f, (size_t)n, nullptr));
            return std::vector<TensorPtr>{op_add_raw(z, g)};
        });
    }
    return out;
}

// ------------------------------------------------------------------ matmul

int g_matmul_mode_override = AKR_MODE_GLOBAL;
// Backward fusion across two autograd nodes (tanh' into the epilogue of the next layer's dA product).
bool g_fuse_backward = true;

// dispatch_matmul of the reference (src/bindings.cpp:1686-1764): forward product plus the autograd
// node. The backward closure calls the fused backward on the original strided operands: no
// transposed copies, no unreduced [batch..., K, N] intermediate, and only the gradients needed.
// True when `t` is the output of a Linear node (x W + b) whose bias wants a gradient: whoever writes the
// gradient of `t` can hand the bias gradient (its column sums) along.
bool feeds_bias_grad(const TensorPtr& t) {
    if (!g_fuse_backward || !t || !t->grad_fn || t->grad_fn->freed || t->grad_fn->op_name != "linear") return false;
    const auto& in = t->grad_fn->inputs;
    return in.size() == 3 && in[2] && in[2]->requires_grad && t->shape.size() >= 2 && t->is_contiguous();
}

TensorPtr op_matmul_bias(const TensorPtr& a, const TensorPtr& b, const TensorPtr& bias) {
    if (a->device != b->device) throw std::runtime_error("Both tensors must be on the same device!");
    require_cuda(a, "matmul");
    if (a->dtype != AKR_DTYPE_F32 || b->dtype != AKR_DTYPE_F32) {
        // float64 / int32 / int64: forward only, as in the reference (src/bindings.cpp:1688-1709)
        if (a->dtype != b->dtype) throw std::runtime_error("matmul: operands must share one dtype");
        if (g_grad_enabled && (a->requires_grad || b->requires_grad))
            throw std::runtime_error(std::string("Autograd is not yet supported for dtype '") + dtype_name(a->dtype) +
                                     "'. Only float32 currently supports gradients.");
        if (bias) throw std::runtime_error("linear: only float32 is supported");
        akr_view ta = a->view(), tb = b->view();
        int64_t ts[AKR_MAX_DIMS + 2];
        int32_t tnd = 0;
        check(akr_matmul_plan(&ta, &tb, ts, &tnd));
        auto typed = std::make_shared<Tensor>(std::vector<int64_t>(ts, ts + tnd), "cuda", a->dtype);
        akr_view tc = typed->view();
        check(akr_matmul_fwd_typed(&ta, &tb, &tc, nullptr));
        return typed;
    }
    akr_view va = a->view(), vb = b->view();
    int64_t oshape[AKR_MAX_DIMS + 2];
    int32_t ond = 0;
    check(akr_matmul_plan(&va, &vb, oshape, &ond));
    auto out = make_cuda(std::vector<int64_t>(oshape, oshape + ond));
    akr_view vo = out->view();
    akr_view vbias;
    if (bias) {
        require_cuda(bias, "matmul bias");
        vbias = bias->view();
    }
    const int mode = g_matmul_mode_override;
    check(akr_matmul_fwd(&va, &vb, bias ? &vbias : nullptr, &vo, mode, nullptr));

    const bool bias_grad = bias && bias->requires_grad;
    if (g_grad_enabled && (a->requires_grad || b->requires_grad || bias_grad)) {
        std::vector<TensorPtr> inputs{a, b};
        if (bias) inputs.push_back(bias);
        auto bw = [a, b, bias, mode](TensorPtr g, bool a_is_tanh) {
            require_cuda(g, "matmul backward");
            TensorPtr da, db, dbias;
            if (a->requires_grad) da = make_cuda(a->shape);
            if (b->requires_grad) db = make_cuda(b->shape);
            akr_view va = a->view(), vb = b->view(), vg = g->view();
            akr_view vda, vdb;
            if (da) vda = da->view();
            if (db) vdb = db->view();
            // The gradient this node produces for `a` flows into the tensor that made `a` (through the tanh when
            // that node is folded in): when that is a Linear output, take its bias gradient in the same launch.
            TensorPtr producer = a;
            if (a_is_tanh && a->grad_fn && !a->grad_fn->inputs.empty()) producer = a->grad_fn->inputs[0];
            if (da && producer->shape == a->shape && feeds_bias_grad(producer)) {
                da->colsum = make_cuda({a->shape.back()});
                check(akr_matmul_bwd_colsum(&va, &vb, &vg, &vda, db ? &vdb : nullptr, da->colsum->data, a_is_tanh ? 1 : 0,
                                            mode, nullptr));
            } else if (da || db) {
                check((a_is_tanh ? akr_matmul_bwd_tanh : akr_matmul_bwd)(&va, &vb, &vg, da ? &vda : nullptr,
                                                                         db ? &vdb : nullptr, mode, nullptr));
            }
            std::vector<TensorPtr> grads{da, db};
            if (bias) {
                if (bias->requires_grad) {
                    // column sums of g: handed along by the kernel that wrote g, else one pass over g
                    if (g->colsum && g->colsum->size == bias->size && g->shape.back() == bias->shape.back()) {
                        dbias = std::make_shared<Tensor>(g->colsum, 0, bias->shape, contiguous_strides(bias->shape));
                    } else {
                        dbias = op_sum_to(g, bias->shape);
                    }
                }
                grads.push_back(dbias);
            }
            return grads;
        };
        attach(out, bias ? "linear" : "matmul", inputs, [bw](TensorPtr g) { return bw(g, false); });
        out->grad_fn->backward_through_tanh = [bw](TensorPtr g) { return bw(g, true); };
    }
    return out;
}

TensorPtr op_matmul(const TensorPtr& a, const TensorPtr& b) { return op_matmul_bias(a, b, nullptr); }

// alpha * (a @ b) + beta * d in one launch; no autograd (used inside optimizer steps).
TensorPtr op_matmul_axpby(const TensorPtr& a, const TensorPtr& b, float alpha, float beta, const TensorPtr& d) {
    require_cuda(a, "matmul_axpby");
    require_f32(a, "matmul_axpby");
    require_cuda(b, "matmul_axpby");
    require_f32(b, "matmul_axpby");
    if (g_grad_enabled && (a->requires_grad || b->requires_grad || (d && d->requires_grad)))
        throw std::runtime_error("matmul_axpby records no gradient: call it under no_grad()");
    akr_view va = a->view(), vb = b->view(), vd;
    if (d) {
        require_cuda(d, "matmul_axpby addend");
        require_f32(d, "matmul_axpby addend");
        vd = d->view();
    }
    int64_t oshape[AKR_MAX_DIMS + 2];
    int32_t ond = 0;
    check(akr_matmul_plan(&va, &vb, oshape, &ond));
    auto out = make_cuda(std::vector<int64_t>(oshape, oshape + ond));
    akr_view vo = out->view();
    check(akr_matmul_fwd_axpby(&va, &vb, alpha, beta, d ? &vd : nullptr, &vo, g_matmul_mode_override, nullptr));
    return out;
}

// mean of squares of a contiguous tensor as a 1-element tensor (no autograd).
TensorPtr op_mean_square(const TensorPtr& t) {
    require_cuda(t, "mean_square");
    require_f32(t, "mean_square");
    auto src = t->is_contiguous() ? t : op_contiguous(t);
    auto out = make_cuda({1});
    check(akr_mse_fwd(src->data, nullptr, out->data, (size_t)src->size, nullptr));
    return out;
}

TensorPtr cpu_matmul_refused(const TensorPtr&, const TensorPtr&) {
    throw std::runtime_error(
        "cpu_matmul: this build computes on CUDA (sm_100a) only; there is no CPU matmul. "
        "Create the tensors with device='cuda'.");
}

// ------------------------------------------------------------------ convolution callers of the matmul path

// im2col_{1,2,3}d and col2im_{1,2,3}d of the reference (dispatch_im2col_1d, src/bindings.cpp:988-1039;
// dispatch_col2im_1d, :1041-1081; the 2-D and 3-D twins up to :1400): unfold into the (B, C*K, L_out) matrix the
// convolution fallback multiplies by the flattened weights, and the adjoint fold that is the forward pass of the
// transposed convolutions. Each is the other's backward. One geometry type (3-D; lower ranks have depth 1).
TensorPtr op_fold(const TensorPtr& col_in, akr_window3d w, int rank, const char* what);

TensorPtr op_unfold(const TensorPtr& x_in, akr_window3d w, int rank, const char* what) {
    require_cuda(x_in, what);
    require_f32(x_in, what);
    auto x = x_in->is_contiguous() ? x_in : op_contiguous(x_in);
    auto col = make_cuda({w.B, w.C * w.KD * w.KH * w.KW, w.OD * w.OH * w.OW});
    check(akr_im2col_3d(x->data, col->data, &w, nullptr));
    if (needs_graph(x)) {
        const auto in_shape = x->shape;
        attach(col, what, {x}, [w, in_shape](TensorPtr g) {
            auto gc = g->is_contiguous() ? g : op_contiguous(g);
            auto gx = make_cuda(in_shape);
            check(akr_col2im_3d(gc->data, gx->data, &w, nullptr));
            return std::vector<TensorPtr>{gx};
        });
    }
    return col;
}

// `rank` spatial dims of the result: (B, C, W), (B, C, H, W) or (B, C, D, H, W).
TensorPtr op_fold(const TensorPtr& col_in, akr_window3d w, int rank, const char* what) {
    require_cuda(col_in, what);
    if (col_in->dtype != AKR_DTYPE_F32) throw std::runtime_error(std::string(what) + ": only float32 is currently supported.");
    auto col = col_in->is_contiguous() ? col_in : op_contiguous(col_in);
    std::vector<int64_t> out_shape{w.B, w.C};
    if (rank == 3) out_shape.push_back(w.D);
    if (rank >= 2) out_shape.push_back(w.H);
    out_shape.push_back(w.W);
    auto out = make_cuda(out_shape);
    check(akr_col2im_3d(col->data, out->data, &w, nullptr));
    if (needs_graph(col)) {
        const auto col_shape = col->shape;
        attach(out, what, {col}, [w, col_shape](TensorPtr g) {
            // the fold's backward is the unfold with the same geometry
            auto gg = g->is_contiguous() ? g : op_contiguous(g);
            auto gc = make_cuda(col_shape);
            check(akr_im2col_3d(gg->data, gc->data, &w, nullptr));
            return std::vector<TensorPtr>{gc};
        });
    }
    return out;
}

akr_window3d window_1d(int64_t B, int64_t C, int64_t L, int K, int S, int P, int D, int64_t L_out) {
    return akr_window3d{B, C, 1, 1, L, 1, 1, K, 1, 1, S, 0, 0, P, 1, 1, D, 1, 1, L_out};
}
akr_window3d window_2d(int64_t B, int64_t C, int64_t H, int64_t W, int KH, int KW, int SH, int SW, int PH, int PW, int DH,
                       int DW, int64_t OH, int64_t OW) {
    return akr_window3d{B, C, 1, H, W, 1, KH, KW, 1, SH, SW, 0, PH, PW, 1, DH, DW, 1, OH, OW};
}

TensorPtr op_im2col_1d(const TensorPtr& x, int K, int S, int P, int D, int64_t L_out) {
    if (x->shape.size() != 3)
        throw std::invalid_argument("im2col_1d: expected input of shape (batch, channels, length), got rank " +
                                    std::to_string(x->shape.size()));
    return op_unfold(x, window_1d(x->shape[0], x->shape[1], x->shape[2], K, S, P, D, L_out), 1, "im2col_1d");
}

TensorPtr op_im2col_2d(const TensorPtr& x, int KH, int KW, int SH, int SW, int PH, int PW, int DH, int DW, int64_t OH,
                       int64_t OW) {
    if (x->shape.size() != 4)
        throw std::invalid_argument("im2col_2d: expected input of shape (batch, channels, H, W), got rank " +
                                    std::to_string(x->shape.size()));
    return op_unfold(x, window_2d(x->shape[0], x->shape[1], x->shape[2], x->shape[3], KH, KW, SH, SW, PH, PW, DH, DW, OH, OW),
                     2, "im2col_2d");
}

TensorPtr op_im2col_3d(const TensorPtr& x, int KD, int KH, int KW, int SD, int SH, int SW, int PD, int PH, int PW, int DD,
                       int DH, int DW, int64_t OD, int64_t OH, int64_t OW) {
    if (x->shape.size() != 5)
        throw std::invalid_argument("im2col_3d: expected input of shape (batch, channels, D, H, W), got rank " +
                                    std::to_string(x->shape.size()));
    akr_window3d w{x->shape[0], x->shape[1], x->shape[2], x->shape[3], x->shape[4], KD, KH, KW, SD, SH, SW,
                   PD, PH, PW, DD, DH, DW, OD, OH, OW};
    return op_unfold(x, w, 3, "im2col_3d");
}

// The reference derives the kernel size from the row count and assumes equal sizes per dim
// (src/bindings.cpp:1094-1099, 1138-1143); explicit sizes (k* > 0) lift that restriction.
int kernel_from_rows(const TensorPtr& col, int64_t C, int dims, const char* what) {
    if (col->shape.size() != 3)
        throw std::invalid_argument(std::string(what) + ": expected input of shape (batch, channels*kernel, positions), got rank " +
                                    std::to_string(col->shape.size()));
    const int64_t rows = col->shape[1];
    if (C <= 0 || rows % C != 0) throw std::invalid_argument(std::string(what) + ": channels*kernel is not divisible by C");
    const int64_t kk = rows / C;
    if (dims == 1) return (int)kk;
    const int k = (int)std::llround(dims == 2 ? std::sqrt((double)kk) : std::cbrt((double)kk));
    int64_t pw = 1;
    for (int i = 0; i < dims; ++i) pw *= k;
    if (pw != kk) throw std::invalid_argument(std::string(what) + ": kernel is not the same size in every dim; pass kernel_size");
    return k;
}

TensorPtr op_col2im_1d(const TensorPtr& col, int64_t C, int64_t L_in, int S, int P, int D, int64_t L_out) {
    const int K = kernel_from_rows(col, C, 1, "col2im_1d");
    if (col->shape[2] != L_out) throw std::invalid_argument("col2im_1d: column count does not match out_length");
    return op_fold(col, window_1d(col->shape[0], C, L_in, K, S, P, D, L_out), 1, "col2im_1d");
}

TensorPtr op_col2im_2d(const TensorPtr& col, int64_t C, int64_t H_in, int64_t W_in, int SH, int SW, int PH, int PW, int DH,
                       int DW, int64_t OH, int64_t OW, int KH, int KW) {
    if (KH <= 0 || KW <= 0) KH = KW = kernel_from_rows(col, C, 2, "col2im_2d");
    if (col->shape.size() != 3 || col->shape[1] != C * KH * KW || col->shape[2] != OH * OW)
        throw std::invalid_argument("col2im_2d: expected input of shape (batch, channels*KH*KW, OH*OW)");
    return op_fold(col, window_2d(col->shape[0], C, H_in, W_in, KH, KW, SH, SW, PH, PW, DH, DW, OH, OW), 2, "col2im_2d");
}

TensorPtr op_col2im_3d(const TensorPtr& col, int64_t C, int64_t D_in, int64_t H_in, int64_t W_in, int SD, int SH, int SW,
                       int PD, int PH, int PW, int DD, int DH, int DW, int64_t OD, int64_t OH, int64_t OW, int KD, int KH,
                       int KW) {
    if (KD <= 0 || KH <= 0 || KW <= 0) KD = KH = KW = kernel_from_rows(col, C, 3, "col2im_3d");
    if (col->shape.size() != 3 || col->shape[1] != C * KD * KH * KW || col->shape[2] != OD * OH * OW)
        throw std::invalid_argument("col2im_3d: expected input of shape (batch, channels*KD*KH*KW, OD*OH*OW)");
    akr_window3d w{col->shape[0], C, D_in, H_in, W_in, KD, KH, KW, SD, SH, SW, PD, PH, PW, DD, DH, DW, OD, OH, OW};
    return op_fold(col, w, 3, "col2im_3d");
}

// ------------------------------------------------------------------ losses / optimiser

// _mse_fused of the reference (src/bindings.cpp:2821, src/elementwise_kernel.cu:2253-2300).
TensorPtr op_mse(const TensorPtr& pred, const TensorPtr& target) {
    require_cuda(pred, "mse");
    require_f32(pred, "mse");
    require_cuda(target, "mse");
    require_f32(target, "mse");
    if (pred->shape != target->shape) throw std::invalid_argument("MSELoss: pred and target shapes differ");
    if (!pred->is_contiguous() || !target->is_contiguous())
        throw std::invalid_argument("MSELoss requires contiguous tensors. Call .contiguous() first.");
    auto out = make_cuda({1});
    if (needs_graph(pred)) {
        // The gradient for an incoming gradient of 1 is written in the forward pass; backward() from this loss
        // (its usual place, the root) then has nothing left to compute.
        auto dp1 = make_cuda(pred->shape);
        if (feeds_bias_grad(pred)) {
            // pred = x W + b: the bias gradient is the column sum of this gradient, taken in the same pass
            const int64_t cols = pred->shape.back();
            dp1->colsum = make_cuda({cols});
            check(akr_mse_fwd_grad_colsum(pred->data, target->data, out->data, dp1->data, dp1->colsum->data,
                                          pred->size / cols, cols, nullptr));
        } else {
            check(akr_mse_fwd_grad(pred->data, target->data, out->data, dp1->data, (size_t)pred->size, nullptr));
        }
        attach(out, "mse", {pred}, [pred, target, dp1](TensorPtr g) {
            if (g.get() == g_unit_root_grad) return std::vector<TensorPtr>{dp1};
            auto dp = make_cuda(pred->shape);
            check(akr_mse_bwd(pred->data, target->data, g->data, dp->data, (size_t)pred->size, nullptr));
            return std::vector<TensorPtr>{dp};
        });
    } else {
        check(akr_mse_fwd(pred->data, target->data, out->data, (size_t)pred->size, nullptr));
    }
    return out;
}

void op_sgd_step(const TensorPtr& p, const TensorPtr& grad, const TensorPtr& velocity, float lr,
                 float momentum, float weight_decay, float dampening, int nesterov, int has_momentum,
                 int velocity_initialized) {
    require_cuda(p, "sgd_step");
    require_f32(p, "sgd_step");
    require_cuda(grad, "sgd_step");
    require_f32(grad, "sgd_step");
    if (!p->is_contiguous() || !grad->is_contiguous())
        throw std::invalid_argument("sgd_step requires contiguous tensors");
    if (p->size != grad->size) throw std::invalid_argument("sgd_step: parameter and gradient sizes differ");
    check(akr_sgd_step(p->data, grad->data, velocity ? velocity->data : nullptr, lr, momentum, weight_decay,
                       dampening, nesterov, has_momentum, velocity_initialized, (size_t)p->size, nullptr));
}

// SGD.step over a parameter list in one launch (contiguous float32 CUDA tensors; the caller filters).
void op_sgd_step_multi(const std::vector<TensorPtr>& params, const std::vector<TensorPtr>& grads,
                       const std::vector<TensorPtr>& velocities, const std::vector<int>& vel_init, float lr,
                       float momentum, float weight_decay, float dampening, int nesterov, int has_momentum) {
    const size_t n = params.size();
    if (grads.size() != n || vel_init.size() != n || (has_momentum && velocities.size() != n))
        throw std::invalid_argument("sgd_step_multi: list lengths differ");
    std::vector<float*> pp(n), vv(n);
    std::vector<const float*> gg(n);
    std::vector<size_t> sz(n);
    for (size_t i = 0; i < n; ++i) {
        require_cuda(params[i], "sgd_step");
        require_f32(params[i], "sgd_step");
        require_cuda(grads[i], "sgd_step");
        if (!params[i]->is_contiguous() || !grads[i]->is_contiguous())
            throw std::invalid_argument("sgd_step requires contiguous tensors");
        if (params[i]->size != grads[i]->size) throw std::invalid_argument("sgd_step: parameter and gradient sizes differ");
        pp[i] = params[i]->data;
        gg[i] = grads[i]->data;
        vv[i] = has_momentum ? velocities[i]->data : nullptr;
        sz[i] = (size_t)params[i]->size;
    }
    check(akr_sgd_step_multi((int)n, pp.data(), gg.data(), has_momentum ? vv.data() : nullptr, sz.data(), vel_init.data(),
                             lr, momentum, weight_decay, dampening, nesterov, has_momentum, nullptr));
}

// ------------------------------------------------------------------ backward driver
// tensor_backward of the reference (src/bindings.cpp:810-877): reverse topological walk, leaf
// gradients accumulate with add, a graph can be walked once unless retain_graph is set.
void tensor_backward(const TensorPtr& root, TensorPtr grad_output, bool retain_graph) {
    if (!grad_output) {
        if (root->size != 1)
            throw std::runtime_error("backward() requires an explicit gradient for non-scalar tensors");
        require_cuda(root, "backward");
        grad_output = make_cuda(root->shape);
        check(akr_fill(grad_output->data, 1.0f, 1, nullptr));
        g_unit_root_grad = grad_output.get();
    }
    std::vector<TensorPtr> topo;
    std::unordered_set<Tensor*> seen;
    // Iterative post-order DFS (deep graphs must not overflow the C stack).
    std::vector<std::pair<TensorPtr, size_t>> stack;
    stack.emplace_back(root, 0);
    seen.insert(root.get());
    while (!stack.empty()) {
        auto& top = stack.back();
        TensorPtr t = top.first;
        if (t->grad_fn && top.second < t->grad_fn->inputs.size()) {
            TensorPtr nxt = t->grad_fn->inputs[top.second++];
            if (nxt && !seen.count(nxt.get())) {
                seen.insert(nxt.get());
                stack.emplace_back(nxt, 0);
            }
        } else {
            topo.push_back(t);
            stack.pop_back();
        }
    }
    // How many nodes of this graph consume each tensor: a tanh output that feeds exactly one matmul can
    // have its backward folded into that matmul's.
    std::unordered_map<Tensor*, int> uses;
    for (const TensorPtr& t : topo)
        if (t->grad_fn)
            for (const TensorPtr& inp : t->grad_fn->inputs)
                if (inp) ++uses[inp.get()];
    const bool prev = g_grad_enabled;
    g_grad_enabled = false;  // gradient arithmetic is not itself recorded
    try {
        std::unordered_map<Tensor*, TensorPtr> grads;
        grads[root.get()] = grad_output;
        for (auto it = topo.rbegin(); it != topo.rend(); ++it) {
            const TensorPtr& t = *it;
            auto found = grads.find(t.get());
            if (found == grads.end()) continue;
            TensorPtr g = found->second;
            if (t->requires_grad && !t->grad_fn) {
                t->grad = t->grad ? op_add_raw(t->grad, g) : g;
            }
            if (t->grad_fn) {
                if (t->grad_fn->freed)
                    throw std::runtime_error(
                        "Trying to backward through the graph a second time (or a part of it), but the "
                        "intermediate results needed have already been freed. Pass retain_graph=True to "
                        "backward() the first time if you need to backward through this part of the graph "
                        "more than once.");
                // tanh -> matmul: when this node's first input is a tanh output nobody else consumes, ask for
                // the gradient with respect to the tanh's INPUT directly and skip the tanh node.
                TensorPtr through;
                if (g_fuse_backward && t->grad_fn->backward_through_tanh && !t->grad_fn->inputs.empty()) {
                    const TensorPtr& h = t->grad_fn->inputs[0];
                    if (h && h.get() != root.get() && h->requires_grad && h->grad_fn && !h->grad_fn->freed &&
                        h->grad_fn->op_name == "tanh" && uses[h.get()] == 1 && !grads.count(h.get()) &&
                        h->grad_fn->inputs.size() == 1 && h->grad_fn->inputs[0] && h->grad_fn->inputs[0]->requires_grad)
                        through = h->grad_fn->inputs[0];
                }
                auto in_grads = through ? t->grad_fn->backward_through_tanh(g) : t->grad_fn->backward_fn(g);
                for (size_t i = 0; i < t->grad_fn->inputs.size(); ++i) {
                    const TensorPtr& inp = (through && i == 0) ? through : t->grad_fn->inputs[i];
                    if (!inp || !inp->requires_grad || i >= in_grads.size() || !in_grads[i]) continue;
                    auto ex = grads.find(inp.get());
                    if (ex == grads.end()) grads[inp.get()] = in_grads[i];
                    else ex->second = op_add_raw(ex->second, in_grads[i]);
                }
            }
        }
    } catch (...) {
        g_grad_enabled = prev;
        g_unit_root_grad = nullptr;
        throw;
    }
    g_grad_enabled = prev;
    g_unit_root_grad = nullptr;
    if (!retain_graph)
        for (auto& t : topo)
            if (t->grad_fn) t->grad_fn->freed = true;
}

// ------------------------------------------------------------------ host <-> device

TensorPtr from_numpy(py::array array, const std::string& device, bool requires_grad) {
    int dt;
    if (py::isinstance<py::array_t<float>>(array)) dt = AKR_DTYPE_F32;
    else if (py::isinstance<py::array_t<double>>(array)) dt = AKR_DTYPE_F64;
    else if (py::isinstance<py::array_t<int32_t>>(array)) dt = AKR_DTYPE_I32;
    else if (py::isinstance<py::array_t<int64_t>>(array)) dt = AKR_DTYPE_I64;
    else
        throw std::runtime_error("from_numpy: unsupported dtype " + std::string(py::str(array.dtype())) +
                                 " (float32, float64, int32 and int64 are accepted)");
    if (dt != AKR_DTYPE_F32 && requires_grad)
        throw std::runtime_error(std::string("Autograd is not yet supported for dtype '") + dtype_name(dt) +
                                 "'. Only float32 currently supports gradients.");
    py::array arr = py::array::ensure(array, py::array::c_style);
    if (!arr) throw std::runtime_error("from_numpy: could not read the array as C-contiguous");
    std::vector<int64_t> shape(arr.ndim());
    for (py::ssize_t i = 0; i < arr.ndim(); ++i) shape[i] = arr.shape(i);
    if (shape.empty()) shape.push_back(1);
    auto t = std::make_shared<Tensor>(shape, device, dt);
    if (device == "cuda") {
        check(akr_memcpy_h2d(t->data, arr.data(), t->nbytes(), nullptr));
        // the source may be freed by the caller right after this returns
        check(akr_stream_synchronize(nullptr));
    } else {
        std::memcpy(t->data, arr.data(), t->nbytes());
    }
    t->requires_grad = requires_grad;
    return t;
}

// Asynchronous upload from page-locked memory: returns as soon as the copy is queued. The caller
// keeps `array` alive and unchanged until the next synchronize().
TensorPtr from_pinned(py::array_t<float, py::array::c_style> arr, bool requires_grad) {
    std::vector<int64_t> shape(arr.ndim());
    for (py::ssize_t i = 0; i < arr.ndim(); ++i) shape[i] = arr.shape(i);
    if (shape.empty()) shape.push_back(1);
    auto t = make_cuda(shape);
    check(akr_memcpy_h2d(t->data, arr.data(), (size_t)t->size * sizeof(float), nullptr));
    t->requires_grad = requires_grad;
    return t;
}

py::array to_numpy(const TensorPtr& t) {
    std::vector<py::ssize_t> shape(t->shape.begin(), t->shape.end());
    py::array out;
    switch (t->dtype) {
        case AKR_DTYPE_F64: out = py::array_t<double>(shape); break;
        case AKR_DTYPE_I32: out = py::array_t<int32_t>(shape); break;
        case AKR_DTYPE_I64: out = py::array_t<int64_t>(shape); break;
        default: out = py::array_t<float>(shape); break;
    }
    if (t->device == "cuda") {
        bool prev = g_grad_enabled;
        g_grad_enabled = false;
        TensorPtr src = t->is_contiguous() ? t : op_contiguous(t);   // gather is float32-only
        g_grad_enabled = prev;
        check(akr_memcpy_d2h(out.mutable_data(), src->data, t->nbytes(), nullptr));
        check(akr_synchronize());
    } else {
        if (!t->is_contiguous()) throw std::runtime_error("to_numpy: non-contiguous CPU tensors are not supported");
        std::memcpy(out.mutable_data(), t->data, t->nbytes());
    }
    return out;
}

// Download into caller-provided (ideally page-locked) memory without synchronising.
void copy_to_host(const TensorPtr& t, py::array_t<float, py::array::c_style> out) {
    require_cuda(t, "copy_to_host");
    require_f32(t, "copy_to_host");
    if ((int64_t)out.size() != t->size) throw std::invalid_argument("copy_to_host: size mismatch");
    bool prev = g_grad_enabled;
    g_grad_enabled = false;
    TensorPtr src = t->is_contiguous() ? t : op_contiguous(t);
    g_grad_enabled = prev;
    check(akr_memcpy_d2h(out.mutable_data(), src->data, (size_t)t->size * sizeof(float), nullptr));
}

py::array_t<float> pinned_empty(const std::vector<int64_t>& shape) {
    size_t n = 1;
    for (auto d : shape) n *= (size_t)d;
    void* p = nullptr;
    check(akr_host_alloc(n * sizeof(float), &p));
    py::capsule owner(p, [](void* q) { akr_host_free(q); });
    std::vector<py::ssize_t> shp(shape.begin(), shape.end());
    return py::array_t<float>(shp, static_cast<float*>(p), owner);
}

TensorPtr to_device(const TensorPtr& t, const std::string& target) {
    if (target == t->device) return t;
    if (target != "cuda" && target != "cpu") throw std::invalid_argument("Unknown device '" + target + "'");
    auto out = std::make_shared<Tensor>(t->shape, target, t->dtype);
    const size_t bytes = t->nbytes();
    if (target == "cuda") {
        if (!t->is_contiguous()) throw std::runtime_error("to('cuda'): CPU tensor must be contiguous");
        check(akr_memcpy_h2d(out->data, t->data, bytes, nullptr));
        check(akr_stream_synchronize(nullptr));
    } else {
        bool prev = g_grad_enabled;
        g_grad_enabled = false;
        TensorPtr src = t->is_contiguous() ? t : op_contiguous(t);
        g_grad_enabled = prev;
        check(akr_memcpy_d2h(out->data, src->data, bytes, nullptr));
        check(akr_synchronize());
    }
    out->requires_grad = t->requires_grad;
    return out;
}

void copy_into(const TensorPtr& dst, const TensorPtr& src) {
    if (dst->size != src->size) throw std::invalid_argument("copy_: size mismatch");
    require_cuda(dst, "copy_");
    require_f32(dst, "copy_");
    bool prev = g_grad_enabled;
    g_grad_enabled = false;
    TensorPtr s = src->is_contiguous() ? src : op_contiguous(src);
    g_grad_enabled = prev;
    if (!dst->is_contiguous()) {
        // a view (transposed, sliced): the dense source is written through the view's strides
        if (s->device != "cuda") throw std::invalid_argument("copy_: a non-contiguous destination takes a CUDA source");
        akr_view vd = dst->view();
        check(akr_scatter(s->data, &vd, nullptr));
        return;
    }
    if (s->device == "cuda") check(akr_memcpy_d2d(dst->data, s->data, (size_t)dst->size * sizeof(float), nullptr));
    else {
        check(akr_memcpy_h2d(dst->data, s->data, (size_t)dst->size * sizeof(float), nullptr));
        check(akr_stream_synchronize(nullptr));
    }
}

float item(const TensorPtr& t) {
    require_f32(t, "item");
    if (t->size != 1) throw std::runtime_error("item() only works on tensors with exactly one element");
    float v = 0.f;
    if (t->device == "cuda") {
        check(akr_memcpy_d2h(&v, t->data, sizeof(float), nullptr));
        check(akr_synchronize());
    } else {
        v = t->data[0];
    }
    return v;
}

// Basic indexing: ints, slices and tuples of them produce a view (offset + scaled strides), as
// Tensor.__getitem__ of the reference does (src/bindings.cpp:2613-2732). The node's backward places the
// incoming gradient into a zero tensor of the base's shape, at the positions the view covers.
TensorPtr getitem(const TensorPtr& self, py::object key) {
    py::tuple keys = py::isinstance<py::tuple>(key) ? key.cast<py::tuple>() : py::make_tuple(key);
    if (keys.size() > self->shape.size()) throw std::out_of_range("too many indices for tensor");
    std::vector<int64_t> shape, strides;
    int64_t off = 0;
    size_t dim = 0;
    for (auto k : keys) {
        const int64_t extent = self->shape[dim], st = self->strides[dim];
        if (py::isinstance<py::slice>(k)) {
            py::ssize_t start, stop, step, len;
            if (!k.cast<py::slice>().compute(extent, &start, &stop, &step, &len)) throw py::error_already_set();
            if (step <= 0) throw std::invalid_argument("slice step must be positive");
            if (len <= 0) throw std::invalid_argument("Tensor dimensions must be positive");
            off += start * st;
            shape.push_back(len);
            strides.push_back(st * step);
        } else if (py::isinstance<py::int_>(k)) {
            int64_t i = k.cast<int64_t>();
            if (i < 0) i += extent;
            if (i < 0 || i >= extent) throw std::out_of_range("index out of range");
            off += i * st;
        } else {
            throw std::invalid_argument("unsupported index type (ints and slices only)");
        }
        ++dim;
    }
    for (; dim < self->shape.size(); ++dim) {
        shape.push_back(self->shape[dim]);
        strides.push_back(self->strides[dim]);
    }
    if (shape.empty()) {
        shape.push_back(1);
        strides.push_back(1);
    }
    auto out = std::make_shared<Tensor>(self, off, shape, strides);
    if (needs_graph(self)) {
        require_f32(self, "__getitem__");
        const auto base_shape = self->shape;
        // the view's geometry relative to a CONTIGUOUS tensor of the base's shape (the gradient is contiguous)
        const auto cst = contiguous_strides(self->shape);
        std::vector<int64_t> gstrides;
        int64_t goff = 0;
        {
            size_t d = 0;
            for (auto k : keys) {
                if (py::isinstance<py::slice>(k)) {
                    py::ssize_t start, stop, step, len;
                    k.cast<py::slice>().compute(self->shape[d], &start, &stop, &step, &len);
                    goff += start * cst[d];
                    gstrides.push_back(cst[d] * step);
                } else {
                    int64_t i = k.cast<int64_t>();
                    if (i < 0) i += self->shape[d];
                    goff += i * cst[d];
                }
                ++d;
            }
            for (; d < self->shape.size(); ++d) gstrides.push_back(cst[d]);
            if (gstrides.empty()) gstrides.push_back(1);
        }
        const auto vshape = shape;
        attach(out, "getitem", {self}, [base_shape, vshape, gstrides, goff](TensorPtr g) {
            require_cuda(g, "__getitem__ backward");
            auto gc = g->is_contiguous() ? g : op_contiguous(g);
            auto gi = make_cuda(base_shape);
            check(akr_fill(gi->data, 0.0f, (size_t)gi->size, nullptr));
            Tensor window(gi, goff, vshape, gstrides);
            akr_view vw = window.view();
            check(akr_scatter(gc->data, &vw, nullptr));
            return std::vector<TensorPtr>{gi};
        });
    }
    return out;
}

std::string repr(const TensorPtr& t) {
    std::ostringstream os;
    os << "Tensor(shape=[";
    for (size_t i = 0; i < t->shape.size(); ++i) os << (i ? ", " : "") << t->shape[i];
    os << "], device='" << t->device << "', dtype=" << dtype_name(t->dtype) << (t->requires_grad ? ", requires_grad=True" : "") << ")";
    return os.str();
}

}  // namespace

PYBIND11_MODULE(_C, m) {
    m.doc() = "aakaar_b200: B200-native fp32 matmul path behind the Aakaar API";

    // DType of the reference (src/dtype.h:6, bound at src/bindings.cpp:2473-2477).
    py::enum_<DTypeEnum>(m, "DType")
        .value("float32", DTypeEnum::float32)
        .value("float64", DTypeEnum::float64)
        .value("int32", DTypeEnum::int32)
        .value("int64", DTypeEnum::int64);

    py::class_<Tensor, TensorPtr>(m, "Tensor")
        .def(py::init([](std::vector<int64_t> shape, std::string device) {
                 return std::make_shared<Tensor>(shape, device);
             }),
             py::arg("shape"), py::arg("device") = "cuda")
        .def(py::init([](std::vector<int64_t> shape, std::string device, DTypeEnum dt) {
                 return std::make_shared<Tensor>(shape, device, (int)dt);
             }),
             py::arg("shape"), py::arg("device"), py::arg("dtype"))
        .def_property_readonly("dtype", [](Tensor& t) { return std::string(dtype_name(t.dtype)); })
        .def_readonly("device", &Tensor::device)
        .def_readonly("size", &Tensor::size)
        .def_readonly("shape", &Tensor::shape)
        .def_readonly("strides", &Tensor::strides)
        .def_readwrite("requires_grad", &Tensor::requires_grad)
        .def_property(
            "grad", [](Tensor& t) { return t.grad; }, [](Tensor& t, TensorPtr g) { t.grad = g; })
        .def_property_readonly("is_leaf", [](Tensor& t) { return !t.grad_fn; })
        .def_property_readonly("data_ptr", [](Tensor& t) { return (uintptr_t)t.data; })
        .def_property_readonly("__cuda_array_interface__",
                               [](Tensor& t) {
                                   if (t.device != "cuda") throw std::runtime_error("not a CUDA tensor");
                                   py::dict d;
                                   d["shape"] = py::tuple(py::cast(t.shape));
                                   d["typestr"] = "<f4";
                                   d["data"] = py::make_tuple((uintptr_t)t.data, false);
                                   d["version"] = 3;
                                   std::vector<int64_t> bs(t.strides.size());
                                   for (size_t i = 0; i < bs.size(); ++i) bs[i] = t.strides[i] * 4;
                                   d["strides"] = py::tuple(py::cast(bs));
                                   return d;
                               })
        .def("to_numpy", &to_numpy)
        .def("copy_to_host", &copy_to_host)
        .def("is_contiguous", &Tensor::is_contiguous)
        .def("contiguous", &op_contiguous)
        .def("tanh", &op_tanh)
        .def("copy_", [](TensorPtr self, TensorPtr src) { copy_into(self, src); return self; })
        .def("to", &to_device)
        .def("to_device", &to_device)
        .def("transpose", &op_transpose)
        .def("transpose2d", [](TensorPtr self) { return op_transpose(self, -2, -1); })
        .def_property_readonly("T", [](TensorPtr self) { return op_transpose(self, -2, -1); })
        .def("backward", &tensor_backward, py::arg("grad_output") = nullptr, py::arg("retain_graph") = false)
        .def("zero_grad", [](Tensor& t) { t.grad = nullptr; })
        .def("item", &item)
        .def("detach",
             [](TensorPtr self) { return std::make_shared<Tensor>(self, 0, self->shape, self->strides); })
        .def("__repr__", &repr)
        .def("__str__", &repr)
        .def("__len__", [](Tensor& t) { return t.shape.empty() ? (int64_t)0 : t.shape[0]; })
        .def("view", [](TensorPtr self, std::vector<int64_t> s) { return op_view(self, s, false); })
        .def("reshape", [](TensorPtr self, std::vector<int64_t> s) { return op_view(self, s, true); })
        .def("sum", [](TensorPtr self) { return op_sum_all(self); })
        .def("__getitem__", &getitem)
        .def("__neg__", [](TensorPtr a) { return op_scale(a, -1.0f); })
        .def("__add__", [](TensorPtr a, TensorPtr b) { return op_add(a, b); })
        .def("__add__", [](TensorPtr a, float s) { return op_add(a, scalar_tensor(s)); })
        .def("__radd__", [](TensorPtr a, float s) { return op_add(a, scalar_tensor(s)); })
        .def("__sub__", [](TensorPtr a, TensorPtr b) { return op_sub(a, b); })
        .def("__sub__", [](TensorPtr a, float s) { return op_add(a, scalar_tensor(-s)); })
        .def("__mul__", [](TensorPtr a, TensorPtr b) { return op_mul(a, b); })
        .def("__mul__", [](TensorPtr a, float s) { return op_scale(a, s); })
        .def("__rmul__", [](TensorPtr a, float s) { return op_scale(a, s); })
        .def("__truediv__", [](TensorPtr a, float s) { return op_scale(a, 1.0f / s); })
        .def("__matmul__", &op_matmul);

    m.def("_set_grad_enabled", [](bool e) { g_grad_enabled = e; });
    m.def("_set_backward_fusion", [](bool e) { g_fuse_backward = e; },
          "tanh' folded into the next matmul's dA epilogue during backward (default on)");
    m.def("_is_grad_enabled", []() { return g_grad_enabled; });
    m.def("cuda_matmul", &op_matmul, "tcgen05 GPU matrix multiplication (autograd-aware)");
    m.def("cpu_matmul", &cpu_matmul_refused, "not available: this build has no CPU matmul");
    m.def("matmul_axpby", &op_matmul_axpby, py::arg("a"), py::arg("b"), py::arg("alpha") = 1.0f, py::arg("beta") = 0.0f,
          py::arg("d") = nullptr, "alpha * (a @ b) + beta * d in one launch (no autograd)");
    m.def("_mean_square", &op_mean_square);
    m.def("im2col_1d", &op_im2col_1d, py::arg("x"), py::arg("kernel_size"), py::arg("stride"), py::arg("padding"),
          py::arg("dilation"), py::arg("out_length"));
    m.def("im2col_2d", &op_im2col_2d);
    m.def("im2col_3d", &op_im2col_3d);
    m.def("col2im_1d", &op_col2im_1d, py::arg("col"), py::arg("C"), py::arg("L_in"), py::arg("stride"), py::arg("padding"),
          py::arg("dilation"), py::arg("out_length"));
    m.def("col2im_2d", &op_col2im_2d, py::arg("col"), py::arg("C"), py::arg("H_in"), py::arg("W_in"), py::arg("SH"),
          py::arg("SW"), py::arg("PH"), py::arg("PW"), py::arg("DH"), py::arg("DW"), py::arg("OH"), py::arg("OW"),
          py::arg("KH") = 0, py::arg("KW") = 0);
    m.def("col2im_3d", &op_col2im_3d, py::arg("col"), py::arg("C"), py::arg("D_in"), py::arg("H_in"), py::arg("W_in"),
          py::arg("SD"), py::arg("SH"), py::arg("SW"), py::arg("PD"), py::arg("PH"), py::arg("PW"), py::arg("DD"),
          py::arg("DH"), py::arg("DW"), py::arg("OD"), py::arg("OH"), py::arg("OW"), py::arg("KD") = 0, py::arg("KH") = 0,
          py::arg("KW") = 0);
    m.def("linear", &op_matmul_bias, py::arg("x"), py::arg("weight"), py::arg("bias") = nullptr,
          "x @ weight + bias with the bias add fused into the GEMM epilogue");
    m.def("from_numpy", &from_numpy, py::arg("array"), py::arg("device") = "cuda", py::arg("requires_grad") = false);
    m.def("from_pinned", &from_pinned, py::arg("array"), py::arg("requires_grad") = false);
    m.def("pinned_empty", &pinned_empty, py::arg("shape"));
    m.def("is_available", []() { return akr_device_count() > 0; });
    m.def("device_count", []() { return akr_device_count(); });
    m.def("set_device", [](int d) { check(akr_set_device(d)); });
    m.def("empty_cache", []() { check(akr_empty_cache()); });
    m.def("_set_tf32_enabled", [](bool e) { akr_set_tf32(e ? 1 : 0); });
    m.def("_get_tf32_enabled", []() { return akr_get_tf32() != 0; });
    m.def("_set_cudnn_tf32_enabled", [](bool e) { akr_set_cudnn_tf32(e ? 1 : 0); });
    m.def("_get_cudnn_tf32_enabled", []() { return akr_get_cudnn_tf32() != 0; });
    m.def("_synchronize", []() { check(akr_synchronize()); });
    m.def("_allocator_stats", []() {
        int64_t h = 0, mi = 0;
        akr_allocator_stats(&h, &mi);
        return py::make_tuple(h, mi);
    });
    m.def("_workspace_bytes", []() {
        size_t b = 0;
        akr_workspace_bytes(&b);
        return b;
    });
    m.def("_launch_count", [](bool reset) { return akr_launch_count(reset ? 1 : 0); }, py::arg("reset") = false);
    m.def("_mse_fused", &op_mse, py::arg("pred"), py::arg("target"));
    m.def("_sgd_step_fused", &op_sgd_step);
    m.def("_sgd_step_multi", &op_sgd_step_multi);
    m.def("_empty_like", [](const TensorPtr& t) {
        require_cuda(t, "empty_like");
        return make_cuda(t->shape);
    }, "an uninitialised device tensor of the same shape (no launch): optimizer state that its first step overwrites");
    m.def("_set_matmul_mode", [](int mode) { g_matmul_mode_override = mode; },
          "per-process override of the arithmetic mode: -1 follow set_tf32, 0 fp32-accurate, 1 TF32");
    m.attr("HAS_CUDA") = true;
    m.attr("HAS_CUDNN") = false;
}
