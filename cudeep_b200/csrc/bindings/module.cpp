// pybind11 module `_cudeep_core`: the extension module cuDeep's Python package imports
// (python/cuDeep/_core.py:3-34 in the reference), built on libcudeep_b200.so.
//
// What lies on the dense-contraction path is implemented with the reference's names and
// signatures (src/bindings/module.cpp:84-181, :326-381, :642-694): DType, Layout, Tensor, Stream,
// Event, MemoryPool, conv2d_forward, conv2d_backward_data / _weight, broadcast_add, relu / sigmoid /
// gelu / silu, device_info; plus the additions linear_forward, matmul_nt and matmul_tn.
// Every other name _core.py imports (losses, norms, pooling, optimisers, reductions, unary math)
// exists so that the import succeeds, and raises RuntimeError when called: those operators are
// outside what this library implements.
#include <pybind11/numpy.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include "cudeep/kernels/conv.cuh"
#include "cudeep/kernels/matmul.cuh"
#include "cudeep/memory.cuh"
#include "cudeep/stream.cuh"
#include "cudeep/tensor.cuh"
#include "cudeep_b200.h"

#include <cstdint>
#include <stdexcept>
#include <string>

namespace py = pybind11;
using namespace cudeep;

namespace {

void check_abi(int rc) {
    if (rc != 0) throw std::runtime_error(cudeep_b200_last_error());
}

Tensor contiguous_of(const Tensor& t) { return t.contiguous(); }

Tensor activation(const Tensor& t, int code, const char* name) {
    if (t.dtype() != DType::Float32) throw std::runtime_error(std::string(name) + ": float32 only");
    Tensor in = contiguous_of(t);
    Tensor out(in.shape(), in.dtype(), in.stream());
    check_abi(cudeep_b200_activation_f32(static_cast<const float*>(in.data()), static_cast<float*>(out.data()),
                                         in.numel(), code, in.stream()));
    return out;
}

struct ConvDims {
    int B, IC, IH, IW, OC, KH, KW, SH, SW, PH, PW, OH, OW;
};

// Extents of a convolution from the shapes of its operands.  Everything the kernels and their
// tensor maps will assume is checked here, before any launch: a mismatch must be a Python
// RuntimeError, never a read past the smaller buffer.
ConvDims conv_dims(const char* op, const std::vector<int64_t>& ishape, const std::vector<int64_t>& wshape,
                   const std::vector<int>& stride, const std::vector<int>& padding) {
    const std::string who(op);
    if (ishape.size() != 4 || wshape.size() != 4 || stride.size() != 2 || padding.size() != 2)
        throw std::runtime_error(who + ": expected 4-D input and weight, 2 strides and 2 paddings");
    for (int64_t v : ishape)
        if (v < 1 || v > INT32_MAX) throw std::runtime_error(who + ": input extents must be positive 32-bit values");
    for (int64_t v : wshape)
        if (v < 1 || v > INT32_MAX) throw std::runtime_error(who + ": weight extents must be positive 32-bit values");
    if (wshape[1] != ishape[1])
        throw std::runtime_error(who + ": weight has " + std::to_string(wshape[1]) + " input channels, input has " +
                                 std::to_string(ishape[1]));
    ConvDims d{};
    d.B = static_cast<int>(ishape[0]); d.IC = static_cast<int>(ishape[1]);
    d.IH = static_cast<int>(ishape[2]); d.IW = static_cast<int>(ishape[3]);
    d.OC = static_cast<int>(wshape[0]); d.KH = static_cast<int>(wshape[2]); d.KW = static_cast<int>(wshape[3]);
    d.SH = stride[0]; d.SW = stride[1]; d.PH = padding[0]; d.PW = padding[1];
    if (d.SH <= 0 || d.SW <= 0) throw std::runtime_error(who + ": stride must be positive");
    if (d.PH < 0 || d.PW < 0) throw std::runtime_error(who + ": padding must not be negative");
    if (d.IH + 2 * d.PH < d.KH || d.IW + 2 * d.PW < d.KW)
        throw std::runtime_error(who + ": kernel larger than the padded input");
    d.OH = (d.IH + 2 * d.PH - d.KH) / d.SH + 1;
    d.OW = (d.IW + 2 * d.PW - d.KW) / d.SW + 1;
    return d;
}

void require_same_dtype(const char* op, const Tensor& a, const Tensor& b, const char* what) {
    if (a.dtype() != b.dtype()) throw std::runtime_error(std::string(op) + ": " + what + " must have the input's dtype");
}

void require_grad_output_shape(const char* op, const Tensor& go, const ConvDims& d) {
    const std::vector<int64_t> want{d.B, d.OC, d.OH, d.OW};
    if (go.shape() != want)
        throw std::runtime_error(std::string(op) + ": grad_output must be [" + std::to_string(d.B) + ", " +
                                 std::to_string(d.OC) + ", " + std::to_string(d.OH) + ", " + std::to_string(d.OW) +
                                 "] for these shapes");
}

// A name the reference's Python layer imports but that lies outside this library.
void out_of_scope(py::module_& m, const char* name) {
    std::string n(name);
    m.def(name, [n](py::args, py::kwargs) -> py::object {
        throw std::runtime_error("_cudeep_core." + n +
                                 " is outside the dense-contraction path (matmul, Linear, Conv2d) this "
                                 "library implements");
    });
}

}  // namespace

PYBIND11_MODULE(_cudeep_core, m) {
    m.doc() = "cuDeep core extension, dense-contraction path on NVIDIA B200 (libcudeep_b200)";

    py::enum_<DType>(m, "DType")
        .value("float16", DType::Float16)
        .value("float32", DType::Float32)
        .value("float64", DType::Float64);
    py::enum_<Layout>(m, "Layout").value("NCHW", Layout::NCHW).value("NHWC", Layout::NHWC);

    py::class_<Tensor>(m, "Tensor")
        .def(py::init<const std::vector<int64_t>&, DType>(), py::arg("shape"), py::arg("dtype") = DType::Float32)
        .def("shape", &Tensor::shape)
        .def("strides", &Tensor::strides)
        .def("ndim", &Tensor::ndim)
        .def("numel", &Tensor::numel)
        .def("nbytes", &Tensor::nbytes)
        .def("dtype", &Tensor::dtype)
        .def("is_contiguous", &Tensor::is_contiguous)
        .def("reshape", &Tensor::reshape)
        .def("transpose", &Tensor::transpose, py::arg("dim0"), py::arg("dim1"))
        .def("contiguous", &Tensor::contiguous)
        .def("fill_", &Tensor::fill_)
        .def("zero_", &Tensor::zero_)
        .def("matmul", &Tensor::matmul)
        // Addition: queue this tensor's work on a Stream (the reference has set_stream in C++ only).
        .def("set_stream", [](Tensor& t, const Stream& s) { t.set_stream(s.get()); }, py::arg("stream"),
             py::keep_alive<1, 2>())
        .def("__add__", &Tensor::operator+)
        .def("__sub__", &Tensor::operator-)
        .def("__mul__", &Tensor::operator*)
        .def_static("zeros", &Tensor::zeros, py::arg("shape"), py::arg("dtype") = DType::Float32)
        .def_static("ones", &Tensor::ones, py::arg("shape"), py::arg("dtype") = DType::Float32)
        .def_static("randn", [](const std::vector<int64_t>& shape, DType dtype) { return Tensor::randn(shape, dtype); },
                    py::arg("shape"), py::arg("dtype") = DType::Float32)
        .def("numpy", [](const Tensor& t) -> py::object {
            std::vector<py::ssize_t> shape(t.shape().begin(), t.shape().end());
            if (t.dtype() == DType::Float32) {
                py::array_t<float> out(shape);
                t.to_host(out.mutable_data());
                return std::move(out);
            }
            if (t.dtype() == DType::Float64) {
                py::array_t<double> out(shape);
                t.to_host(out.mutable_data());
                return std::move(out);
            }
            throw std::runtime_error("numpy() unsupported for this dtype");
        })
        .def_static("from_numpy", [](py::array arr) {
            py::array c = py::array::ensure(arr, py::array::c_style);
            py::buffer_info buf = c.request();
            std::vector<int64_t> shape(buf.shape.begin(), buf.shape.end());
            if (buf.format == py::format_descriptor<float>::format())
                return Tensor::from_host(buf.ptr, shape, DType::Float32);
            if (buf.format == py::format_descriptor<double>::format())
                return Tensor::from_host(buf.ptr, shape, DType::Float64);
            throw std::runtime_error("Unsupported numpy dtype");
        })
        .def("__repr__", [](const Tensor& t) {
            std::string s = "cuDeep.Tensor(shape=[";
            for (size_t i = 0; i < t.shape().size(); ++i) s += (i ? ", " : "") + std::to_string(t.shape()[i]);
            s += "], dtype=";
            s += t.dtype() == DType::Float16 ? "float16" : t.dtype() == DType::Float32 ? "float32" : "float64";
            return s + ")";
        });

    py::class_<Stream>(m, "Stream").def(py::init<>()).def("synchronize", &Stream::synchronize);
    py::class_<Event>(m, "Event")
        .def(py::init<>())
        .def("record", [](Event& e) { e.record(nullptr); })
        .def("record", [](Event& e, Stream& s) { e.record(s.get()); }, py::arg("stream"))
        .def("synchronize", &Event::synchronize)
        .def("elapsed_ms", &Event::elapsed_ms);
    py::class_<MemoryPool, std::unique_ptr<MemoryPool, py::nodelete>>(m, "MemoryPool")
        .def_static("instance", &MemoryPool::instance, py::return_value_policy::reference)
        .def("release_cached", &MemoryPool::release_cached)
        .def_property_readonly("allocated_bytes", &MemoryPool::allocated_bytes)
        .def_property_readonly("cached_bytes", &MemoryPool::cached_bytes);

    m.def("relu", [](const Tensor& t) { return activation(t, CUDEEP_B200_EPI_RELU, "relu"); });
    m.def("gelu", [](const Tensor& t) { return activation(t, CUDEEP_B200_EPI_GELU, "gelu"); });
    m.def("silu", [](const Tensor& t) { return activation(t, CUDEEP_B200_EPI_SILU, "silu"); });
    m.def("sigmoid", [](const Tensor& t) { return activation(t, CUDEEP_B200_EPI_SIGMOID, "sigmoid"); });

    m.def("broadcast_add", [](const Tensor& matrix, const Tensor& row) {
        Tensor mat = contiguous_of(matrix), r = contiguous_of(row);
        if (mat.shape().size() != 2 || r.shape().size() != 1 || mat.shape()[1] != r.shape()[0] ||
            mat.dtype() != r.dtype())
            throw std::runtime_error("broadcast_add: requires matrix [N,M] and row [M], got incompatible shapes");
        Tensor out(mat.shape(), mat.dtype(), mat.stream());
        const long long rows = mat.shape()[0];
        const int cols = static_cast<int>(mat.shape()[1]);
        if (mat.dtype() == DType::Float32)
            check_abi(cudeep_b200_broadcast_add_f32(static_cast<const float*>(mat.data()),
                                                    static_cast<const float*>(r.data()),
                                                    static_cast<float*>(out.data()), rows, cols, mat.stream()));
        else if (mat.dtype() == DType::Float64)
            check_abi(cudeep_b200_broadcast_add_f64(static_cast<const double*>(mat.data()),
                                                    static_cast<const double*>(r.data()),
                                                    static_cast<double*>(out.data()), rows, cols, mat.stream()));
        else
            throw std::runtime_error("broadcast_add: unsupported dtype");
        return out;
    }, py::arg("matrix"), py::arg("row"));

    m.def("linear_forward", [](const Tensor& x, const Tensor& weight, py::object bias_obj, int epilogue) {
        Tensor xc = contiguous_of(x), w = contiguous_of(weight);
        if (w.shape().size() != 2 || xc.shape().empty() || xc.shape().back() != w.shape()[1] ||
            xc.dtype() != w.dtype())
            throw std::runtime_error("linear_forward: x[..., in] and weight[out, in] of one dtype expected");
        const int k = static_cast<int>(w.shape()[1]), n = static_cast<int>(w.shape()[0]);
        const int mrows = static_cast<int>(xc.numel() / k);
        std::vector<int64_t> oshape(xc.shape().begin(), xc.shape().end() - 1);
        oshape.push_back(n);
        Tensor out(oshape, xc.dtype(), xc.stream());
        Tensor bias;
        const void* bptr = nullptr;
        if (!bias_obj.is_none()) {
            bias = contiguous_of(bias_obj.cast<Tensor>());
            if (bias.numel() != n || bias.dtype() != xc.dtype())
                throw std::runtime_error("linear_forward: bias must have out_features elements");
            bptr = bias.data();
        }
        const auto epi = static_cast<kernels::GemmEpilogue>(epilogue);
        if (epilogue < 0 || epilogue > 4) throw std::runtime_error("linear_forward: unknown epilogue");
        if (xc.dtype() == DType::Float32)
            kernels::launch_linear_forward(static_cast<const float*>(xc.data()), static_cast<const float*>(w.data()),
                                           static_cast<const float*>(bptr), static_cast<float*>(out.data()), mrows,
                                           n, k, epi, xc.stream());
        else if (xc.dtype() == DType::Float64)
            kernels::launch_linear_forward(static_cast<const double*>(xc.data()),
                                           static_cast<const double*>(w.data()), static_cast<const double*>(bptr),
                                           static_cast<double*>(out.data()), mrows, n, k, epi, xc.stream());
        else
            throw std::runtime_error("linear_forward: unsupported dtype");
        return out;
    }, py::arg("x"), py::arg("weight"), py::arg("bias") = py::none(), py::arg("epilogue") = 0);

    auto matmul_variant = [](const Tensor& a, const Tensor& b, bool tn) {
        if (a.ndim() != 2 || b.ndim() != 2 || a.dtype() != DType::Float32 || b.dtype() != DType::Float32 ||
            !a.is_contiguous() || !b.is_contiguous())
            throw std::runtime_error("matmul_nt / matmul_tn: contiguous 2-D float32 tensors expected");
        const int64_t mm = tn ? a.shape()[1] : a.shape()[0];
        const int64_t kk = tn ? a.shape()[0] : a.shape()[1];
        const int64_t nn = tn ? b.shape()[1] : b.shape()[0];
        if (kk != (tn ? b.shape()[0] : b.shape()[1]))
            throw std::runtime_error("matmul_nt / matmul_tn: inner dimensions do not match");
        Tensor out({mm, nn}, DType::Float32, a.stream());
        auto fn = tn ? kernels::launch_matmul_tn : kernels::launch_matmul_nt;
        fn(static_cast<const float*>(a.data()), static_cast<const float*>(b.data()), static_cast<float*>(out.data()),
           static_cast<int>(mm), static_cast<int>(nn), static_cast<int>(kk), a.stream());
        return out;
    };
    m.def("matmul_nt", [matmul_variant](const Tensor& a, const Tensor& b) { return matmul_variant(a, b, false); });
    m.def("matmul_tn", [matmul_variant](const Tensor& a, const Tensor& b) { return matmul_variant(a, b, true); });

    m.def("conv2d_forward", [](const Tensor& input, const Tensor& weight, py::object bias_obj,
                               std::vector<int> stride, std::vector<int> padding) {
        Tensor inp = contiguous_of(input), w = contiguous_of(weight);
        const ConvDims d = conv_dims("conv2d_forward", inp.shape(), w.shape(), stride, padding);
        require_same_dtype("conv2d_forward", inp, w, "weight");
        Tensor bias;
        const void* bptr = nullptr;
        if (!bias_obj.is_none()) {
            bias = contiguous_of(bias_obj.cast<Tensor>());
            require_same_dtype("conv2d_forward", inp, bias, "bias");
            if (bias.numel() != d.OC) throw std::runtime_error("conv2d_forward: bias must have out_channels elements");
            bptr = bias.data();
        }
        Tensor out({d.B, d.OC, d.OH, d.OW}, inp.dtype(), inp.stream());
        if (inp.dtype() == DType::Float32)
            kernels::launch_conv2d_forward_kernel<float>(
                static_cast<const float*>(inp.data()), static_cast<const float*>(w.data()),
                static_cast<const float*>(bptr), static_cast<float*>(out.data()), d.B, d.IC, d.OC, d.IH, d.IW,
                d.KH, d.KW, d.SH, d.SW, d.PH, d.PW, inp.stream());
        else if (inp.dtype() == DType::Float64)
            kernels::launch_conv2d_forward_kernel<double>(
                static_cast<const double*>(inp.data()), static_cast<const double*>(w.data()),
                static_cast<const double*>(bptr), static_cast<double*>(out.data()), d.B, d.IC, d.OC, d.IH, d.IW,
                d.KH, d.KW, d.SH, d.SW, d.PH, d.PW, inp.stream());
        else
            throw std::runtime_error("conv2d_forward: unsupported dtype");
        return out;
    }, py::arg("input"), py::arg("weight"), py::arg("bias") = py::none(),
       py::arg("stride") = std::vector<int>{1, 1}, py::arg("padding") = std::vector<int>{0, 0});

    m.def("conv2d_backward_data", [](const Tensor& grad_output, const Tensor& weight,
                                     std::vector<int64_t> input_shape, std::vector<int> stride,
                                     std::vector<int> padding) {
        Tensor go = contiguous_of(grad_output), w = contiguous_of(weight);
        const ConvDims d = conv_dims("conv2d_backward_data", input_shape, w.shape(), stride, padding);
        if (go.dtype() != DType::Float32) throw std::runtime_error("conv2d_backward_data: float32 only");
        require_same_dtype("conv2d_backward_data", go, w, "weight");
        require_grad_output_shape("conv2d_backward_data", go, d);
        Tensor gi(input_shape, go.dtype(), go.stream());
        kernels::launch_conv2d_backward_data_kernel<float>(
            static_cast<const float*>(go.data()), static_cast<const float*>(w.data()),
            static_cast<float*>(gi.data()), d.B, d.IC, d.OC, d.IH, d.IW, d.KH, d.KW, d.SH, d.SW, d.PH, d.PW,
            go.stream());
        return gi;
    }, py::arg("grad_output"), py::arg("weight"), py::arg("input_shape"),
       py::arg("stride") = std::vector<int>{1, 1}, py::arg("padding") = std::vector<int>{0, 0});

    m.def("conv2d_backward_weight", [](const Tensor& grad_output, const Tensor& input,
                                       std::vector<int64_t> weight_shape, std::vector<int> stride,
                                       std::vector<int> padding) {
        Tensor go = contiguous_of(grad_output), inp = contiguous_of(input);
        const ConvDims d = conv_dims("conv2d_backward_weight", inp.shape(), weight_shape, stride, padding);
        if (go.dtype() != DType::Float32) throw std::runtime_error("conv2d_backward_weight: float32 only");
        require_same_dtype("conv2d_backward_weight", go, inp, "input");
        require_grad_output_shape("conv2d_backward_weight", go, d);
        Tensor gw(weight_shape, go.dtype(), go.stream());
        kernels::launch_conv2d_backward_weight_kernel<float>(
            static_cast<const float*>(go.data()), static_cast<const float*>(inp.data()),
            static_cast<float*>(gw.data()), d.B, d.IC, d.OC, d.IH, d.IW, d.KH, d.KW, d.SH, d.SW, d.PH, d.PW,
            go.stream());
        return gw;
    }, py::arg("grad_output"), py::arg("input"), py::arg("weight_shape"),
       py::arg("stride") = std::vector<int>{1, 1}, py::arg("padding") = std::vector<int>{0, 0});

    m.def("device_info", []() {
        int device = 0, sms = 0, major = 0, minor = 0;
        size_t total = 0;
        check_abi(cudeep_b200_device_info(&device, &sms, &major, &minor, &total));
        py::dict info;
        info["device"] = device;
        info["compute_capability"] = std::to_string(major) + "." + std::to_string(minor);
        info["total_memory_mb"] = static_cast<long long>(total / (1024 * 1024));
        info["multiprocessors"] = sms;
        info["warp_size"] = 32;
        return info;
    });

    for (const char* name : {"tanh_act", "leaky_relu", "scalar_mul", "div_op", "neg", "exp_op", "log_op", "sqrt_op",
                             "pow_op", "abs_op", "clamp_op", "gt_mask", "sum", "mean", "max", "min",
                             "sum_reduce_rows", "softmax", "mse_loss", "cross_entropy_loss", "max_pool2d",
                             "avg_pool2d", "batchnorm_forward", "layernorm_forward", "activation_backward",
                             "sgd_update", "adam_update", "adamw_update"})
        out_of_scope(m, name);
}
