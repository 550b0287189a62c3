// TensorFlow OpKernel glue for the B200 build of the SM120 matmul op.
//
// Registers the ops the reference's Python layer expects and forwards them to
// the C ABI in include/sm120_c_interface.h:
//   SM120MatMul          attrs transpose_a, transpose_b, T   (src/tensorflow_ops/sm120_ops_fixed.cc:79-158)
//   SM120AdvancedMatMul  the same plus use_tensor_cores, optimization_level: the
//                        op name python/sm120_ops.py:195-202 actually calls and
//                        that no reference source registers
//   SM120DenseFused      act(x . kernel + bias) in one launch, for SM120Dense
//                        (python/sm120_keras_layers.py:159-174 runs three ops)
//   SM120MatMulFP8       float8_e4m3fn inputs, bfloat16 product
//   SM120MatMulGradA/B   the two backward products, and REGISTER_OP_GRADIENT("SM120MatMul")
//                        (src/tensorflow_ops/sm120_gradients.cc:22-212)
//   SM120BiasGrad        column sums of the output gradient (the gradient of the fused bias)
//   SM120FusedActivation the standalone activation (src/tensorflow_ops/sm120_ops.cc:251-326)
// Differences from the reference glue, all deliberate: the shape function
// honours the transposes (the reference's ignores them, :91-99); an unsupported
// dtype is an error instead of silently becoming FLOAT32 (:44-53); T also
// admits bfloat16; float8_e4m3fn inputs have the op SM120MatMulFP8, whose output
// is bfloat16 (unit scales: scaled FP8 products go through the C ABI's descriptor).
//
// This file needs TensorFlow's headers.  Where they are absent it compiles to
// nothing, and it is not part of _sm120_ops.so as built by csrc/Makefile.

#if defined(__has_include)
#if __has_include("tensorflow/core/framework/op.h")
#define SM120_HAVE_TENSORFLOW 1
#endif
#endif

#ifdef SM120_HAVE_TENSORFLOW

#include <string>

#include "tensorflow/core/framework/function.h"
#include "tensorflow/core/framework/op.h"
#include "tensorflow/core/framework/op_kernel.h"
#include "tensorflow/core/framework/shape_inference.h"
#include "tensorflow/core/framework/tensor.h"
#include "tensorflow/core/platform/stream_executor.h"

#include "../../include/sm120_c_interface.h"

namespace tensorflow {
namespace {

template <typename T> struct ToSM120;
template <> struct ToSM120<float> { static constexpr int value = SM120_DTYPE_FLOAT32; };
template <> struct ToSM120<Eigen::half> { static constexpr int value = SM120_DTYPE_FLOAT16; };
template <> struct ToSM120<bfloat16> { static constexpr int value = SM120_DTYPE_BFLOAT16; };
template <> struct ToSM120<float8_e4m3fn> { static constexpr int value = SM120_DTYPE_FP8_E4M3; };
// the product of two FP8 matrices is written as bfloat16
template <typename T> struct OutOf { using type = T; };
template <> struct OutOf<float8_e4m3fn> { using type = bfloat16; };

// The stream TensorFlow runs this op on (src/tensorflow_ops/sm120_ops_fixed.cc:132-133).
cudaStream_t StreamOf(OpKernelContext* ctx) {
  auto* stream = ctx->op_device_context()->stream();
  return stream ? reinterpret_cast<cudaStream_t>(stream->platform_specific_handle().stream) : nullptr;
}

Status MatMulShape(shape_inference::InferenceContext* c) {
  shape_inference::ShapeHandle a, b;
  TF_RETURN_IF_ERROR(c->WithRank(c->input(0), 2, &a));
  TF_RETURN_IF_ERROR(c->WithRank(c->input(1), 2, &b));
  bool ta = false, tb = false;
  TF_RETURN_IF_ERROR(c->GetAttr("transpose_a", &ta));
  TF_RETURN_IF_ERROR(c->GetAttr("transpose_b", &tb));
  shape_inference::DimensionHandle merged;
  TF_RETURN_IF_ERROR(c->Merge(c->Dim(a, ta ? 0 : 1), c->Dim(b, tb ? 1 : 0), &merged));
  c->set_output(0, c->Matrix(c->Dim(a, ta ? 1 : 0), c->Dim(b, tb ? 0 : 1)));
  return OkStatus();
}

int ActivationCode(const std::string& name) {
  if (name.empty() || name == "linear" || name == "none") return SM120_ACTIVATION_NONE;
  if (name == "relu") return SM120_ACTIVATION_RELU;
  if (name == "gelu" || name == "gelu_erf") return SM120_ACTIVATION_GELU_ERF;
  if (name == "gelu_tanh") return SM120_ACTIVATION_GELU;
  if (name == "tanh") return SM120_ACTIVATION_TANH;
  if (name == "sigmoid") return SM120_ACTIVATION_SIGMOID;
  if (name == "swish" || name == "silu") return SM120_ACTIVATION_SWISH;
  if (name == "elu") return SM120_ACTIVATION_ELU;
  if (name == "selu") return SM120_ACTIVATION_SELU;
  if (name == "leaky_relu") return SM120_ACTIVATION_LEAKY_RELU;
  if (name == "mish") return SM120_ACTIVATION_MISH;
  return -2;
}

}  // namespace

REGISTER_OP("SM120MatMul")
    .Input("a: T").Input("b: T").Output("product: T")
    .Attr("transpose_a: bool = false").Attr("transpose_b: bool = false")
    .Attr("T: {float, half, bfloat16}")
    .SetShapeFn(MatMulShape);

REGISTER_OP("SM120AdvancedMatMul")
    .Input("a: T").Input("b: T").Output("product: T")
    .Attr("transpose_a: bool = false").Attr("transpose_b: bool = false")
    .Attr("use_tensor_cores: bool = true").Attr("optimization_level: int = 1")
    .Attr("T: {float, half, bfloat16}")
    .SetShapeFn(MatMulShape);

// FP8 inputs change the output type, so they get an op of their own: product = bfloat16(a . b)
REGISTER_OP("SM120MatMulFP8")
    .Input("a: float8_e4m3fn").Input("b: float8_e4m3fn").Output("product: bfloat16")
    .Attr("transpose_a: bool = false").Attr("transpose_b: bool = false")
    .SetShapeFn(MatMulShape);

// grad_a[M,K] = grad_output[M,N] . b[K,N]^T and grad_b[K,N] = a[M,K]^T . grad_output[M,N], for the op without
// transposes (src/tensorflow_ops/sm120_gradients.cc:58-98)
REGISTER_OP("SM120MatMulGradA")
    .Input("grad_output: T").Input("b: T").Output("grad_a: T")
    .Attr("transpose_a: bool = false").Attr("transpose_b: bool = false")
    .Attr("T: {float, half, bfloat16}")
    .SetShapeFn([](shape_inference::InferenceContext* c) {
      shape_inference::ShapeHandle g, b;
      TF_RETURN_IF_ERROR(c->WithRank(c->input(0), 2, &g));
      TF_RETURN_IF_ERROR(c->WithRank(c->input(1), 2, &b));
      c->set_output(0, c->Matrix(c->Dim(g, 0), c->Dim(b, 0)));
      return OkStatus();
    });

REGISTER_OP("SM120MatMulGradB")
    .Input("a: T").Input("grad_output: T").Output("grad_b: T")
    .Attr("transpose_a: bool = false").Attr("transpose_b: bool = false")
    .Attr("T: {float, half, bfloat16}")
    .SetShapeFn([](shape_inference::InferenceContext* c) {
      shape_inference::ShapeHandle a, g;
      TF_RETURN_IF_ERROR(c->WithRank(c->input(0), 2, &a));
      TF_RETURN_IF_ERROR(c->WithRank(c->input(1), 2, &g));
      c->set_output(0, c->Matrix(c->Dim(a, 1), c->Dim(g, 1)));
      return OkStatus();
    });

REGISTER_OP("SM120BiasGrad")
    .Input("grad_output: T").Output("grad_bias: T")
    .Attr("T: {float, half, bfloat16}")
    .SetShapeFn([](shape_inference::InferenceContext* c) {
      shape_inference::ShapeHandle g;
      TF_RETURN_IF_ERROR(c->WithRank(c->input(0), 2, &g));
      c->set_output(0, c->Vector(c->Dim(g, 1)));
      return OkStatus();
    });

REGISTER_OP("SM120FusedActivation")
    .Input("input: T").Output("output: T")
    .Attr("T: {float, half, bfloat16}").Attr("activation: string")
    .SetShapeFn([](shape_inference::InferenceContext* c) {
      c->set_output(0, c->input(0));
      return OkStatus();
    });

// The gradient of SM120MatMul as two nodes of the ops above (src/tensorflow_ops/sm120_gradients.cc:22-55).
REGISTER_OP_GRADIENT("SM120MatMul", [](const AttrSlice& attrs, FunctionDef* g) {
  // clang-format off
  *g = FunctionDefHelper::Define(
      {"a: T", "b: T", "grad_output: T"}, {"grad_a: T", "grad_b: T"},
      {"T: {float, half, bfloat16}", "transpose_a: bool = false", "transpose_b: bool = false"},
      {{{"grad_a"}, "SM120MatMulGradA", {"grad_output", "b"}, {{"T", "$T"}}},
       {{"grad_b"}, "SM120MatMulGradB", {"a", "grad_output"}, {{"T", "$T"}}}});
  // clang-format on
  return OkStatus();
});

REGISTER_OP("SM120DenseFused")
    .Input("x: T").Input("kernel: T").Input("bias: T").Output("y: T")
    .Attr("activation: string = ''").Attr("T: {float, half, bfloat16}")
    .SetShapeFn([](shape_inference::InferenceContext* c) {
      shape_inference::ShapeHandle x, k;
      TF_RETURN_IF_ERROR(c->WithRank(c->input(0), 2, &x));
      TF_RETURN_IF_ERROR(c->WithRank(c->input(1), 2, &k));
      shape_inference::DimensionHandle merged;
      TF_RETURN_IF_ERROR(c->Merge(c->Dim(x, 1), c->Dim(k, 0), &merged));
      c->set_output(0, c->Matrix(c->Dim(x, 0), c->Dim(k, 1)));
      return OkStatus();
    });

template <typename T>
class SM120MatMulOp : public OpKernel {
 public:
  explicit SM120MatMulOp(OpKernelConstruction* ctx) : OpKernel(ctx) {
    OP_REQUIRES_OK(ctx, ctx->GetAttr("transpose_a", &transpose_a_));
    OP_REQUIRES_OK(ctx, ctx->GetAttr("transpose_b", &transpose_b_));
    if (ctx->HasAttr("use_tensor_cores")) OP_REQUIRES_OK(ctx, ctx->GetAttr("use_tensor_cores", &use_tensor_cores_));
    if (ctx->HasAttr("optimization_level")) OP_REQUIRES_OK(ctx, ctx->GetAttr("optimization_level", &optimization_level_));
    OP_REQUIRES(ctx, optimization_level_ >= 0 && optimization_level_ <= 2,
                errors::InvalidArgument("optimization_level must be 0, 1 or 2"));
  }

  void Compute(OpKernelContext* ctx) override {
    const Tensor& a = ctx->input(0);
    const Tensor& b = ctx->input(1);
    OP_REQUIRES(ctx, a.dims() == 2, errors::InvalidArgument("Matrix A must be 2-dimensional"));
    OP_REQUIRES(ctx, b.dims() == 2, errors::InvalidArgument("Matrix B must be 2-dimensional"));
    const int64_t a_rows = transpose_a_ ? a.dim_size(1) : a.dim_size(0);
    const int64_t a_cols = transpose_a_ ? a.dim_size(0) : a.dim_size(1);
    const int64_t b_rows = transpose_b_ ? b.dim_size(1) : b.dim_size(0);
    const int64_t b_cols = transpose_b_ ? b.dim_size(0) : b.dim_size(1);
    OP_REQUIRES(ctx, a_cols == b_rows, errors::InvalidArgument("Matrix dimensions must be compatible"));
    Tensor* out = nullptr;
    OP_REQUIRES_OK(ctx, ctx->allocate_output(0, TensorShape({a_rows, b_cols}), &out));
    if (out->NumElements() == 0) return;

    using TOut = typename OutOf<T>::type;
    SM120GemmDesc d;
    sm120_gemm_desc_init(&d);
    d.A = a.flat<T>().data();
    d.B = b.flat<T>().data();
    d.C = out->flat<TOut>().data();
    d.M = a_rows; d.N = b_cols; d.K = a_cols;
    d.transpose_a = transpose_a_; d.transpose_b = transpose_b_;
    d.in_dtype = ToSM120<T>::value;
    d.out_dtype = ToSM120<TOut>::value;
    d.path = use_tensor_cores_ ? SM120_PATH_AUTO : SM120_PATH_SIMT;
    d.optimization_level = optimization_level_;
    d.stream = StreamOf(ctx);
    const cudaError_t rc = sm120_launch_matmul_ex(&d);
    OP_REQUIRES(ctx, rc == cudaSuccess, errors::Internal("SM120MatMul failed: ", sm120_get_error_string(rc)));
  }

 private:
  bool transpose_a_ = false, transpose_b_ = false, use_tensor_cores_ = true;
  int optimization_level_ = 1;
};

template <typename T>
class SM120DenseFusedOp : public OpKernel {
 public:
  explicit SM120DenseFusedOp(OpKernelConstruction* ctx) : OpKernel(ctx) {
    std::string name;
    OP_REQUIRES_OK(ctx, ctx->GetAttr("activation", &name));
    activation_ = ActivationCode(name);
    OP_REQUIRES(ctx, activation_ != -2, errors::InvalidArgument("activation '", name, "' is not fused"));
  }

  void Compute(OpKernelContext* ctx) override {
    const Tensor& x = ctx->input(0);
    const Tensor& k = ctx->input(1);
    const Tensor& bias = ctx->input(2);
    OP_REQUIRES(ctx, x.dims() == 2 && k.dims() == 2, errors::InvalidArgument("x and kernel must be 2-dimensional"));
    OP_REQUIRES(ctx, x.dim_size(1) == k.dim_size(0), errors::InvalidArgument("Matrix dimensions must be compatible"));
    OP_REQUIRES(ctx, bias.NumElements() == 0 || (bias.dims() == 1 && bias.dim_size(0) == k.dim_size(1)),
                errors::InvalidArgument("bias must have shape [units]"));
    Tensor* out = nullptr;
    OP_REQUIRES_OK(ctx, ctx->allocate_output(0, TensorShape({x.dim_size(0), k.dim_size(1)}), &out));
    if (out->NumElements() == 0) return;

    SM120GemmDesc d;
    sm120_gemm_desc_init(&d);
    d.A = x.flat<T>().data();
    d.B = k.flat<T>().data();
    d.C = out->flat<T>().data();
    d.M = x.dim_size(0); d.N = k.dim_size(1); d.K = x.dim_size(1);
    d.in_dtype = d.out_dtype = ToSM120<T>::value;
    if (bias.NumElements() != 0) {
      d.bias = bias.flat<T>().data();
      d.bias_dtype = ToSM120<T>::value;
    }
    d.activation = activation_;
    d.stream = StreamOf(ctx);
    const cudaError_t rc = sm120_launch_matmul_ex(&d);
    OP_REQUIRES(ctx, rc == cudaSuccess, errors::Internal("SM120DenseFused failed: ", sm120_get_error_string(rc)));
  }

 private:
  int activation_ = SM120_ACTIVATION_NONE;
};

// grad_a, grad_b and grad_bias through the C ABI's backward entry points.
template <typename T, int WHICH>   // 0: GradA, 1: GradB, 2: BiasGrad
class SM120BackwardOp : public OpKernel {
 public:
  explicit SM120BackwardOp(OpKernelConstruction* ctx) : OpKernel(ctx) {
    if (WHICH != 2) {
      bool ta = false, tb = false;
      OP_REQUIRES_OK(ctx, ctx->GetAttr("transpose_a", &ta));
      OP_REQUIRES_OK(ctx, ctx->GetAttr("transpose_b", &tb));
      OP_REQUIRES(ctx, !ta && !tb, errors::Unimplemented("gradients are implemented for the op without transposes"));
    }
  }

  void Compute(OpKernelContext* ctx) override {
    const Tensor& x = ctx->input(0);
    OP_REQUIRES(ctx, x.dims() == 2, errors::InvalidArgument("inputs must be 2-dimensional"));
    cudaStream_t stream = StreamOf(ctx);
    Tensor* out = nullptr;
    cudaError_t rc = cudaSuccess;
    if (WHICH == 2) {
      OP_REQUIRES_OK(ctx, ctx->allocate_output(0, TensorShape({x.dim_size(1)}), &out));
      rc = sm120_launch_bias_grad(x.flat<T>().data(), out->flat<T>().data(), x.dim_size(0), x.dim_size(1), 0,
                                  static_cast<SM120DataType>(ToSM120<T>::value), static_cast<SM120DataType>(ToSM120<T>::value), stream);
    } else {
      const Tensor& y = ctx->input(1);
      OP_REQUIRES(ctx, y.dims() == 2, errors::InvalidArgument("inputs must be 2-dimensional"));
      if (WHICH == 0) {       // x = grad_output [M,N], y = b [K,N]
        OP_REQUIRES(ctx, x.dim_size(1) == y.dim_size(1), errors::InvalidArgument("Matrix dimensions must be compatible"));
        OP_REQUIRES_OK(ctx, ctx->allocate_output(0, TensorShape({x.dim_size(0), y.dim_size(0)}), &out));
        if (out->NumElements() == 0) return;
        rc = sm120_launch_matmul_grad_a(x.flat<T>().data(), y.flat<T>().data(), out->flat<T>().data(), x.dim_size(0), x.dim_size(1),
                                        y.dim_size(0), 1.0f, static_cast<SM120DataType>(ToSM120<T>::value), stream);
      } else {                // x = a [M,K], y = grad_output [M,N]
        OP_REQUIRES(ctx, x.dim_size(0) == y.dim_size(0), errors::InvalidArgument("Matrix dimensions must be compatible"));
        OP_REQUIRES_OK(ctx, ctx->allocate_output(0, TensorShape({x.dim_size(1), y.dim_size(1)}), &out));
        if (out->NumElements() == 0) return;
        rc = sm120_launch_matmul_grad_b(x.flat<T>().data(), y.flat<T>().data(), out->flat<T>().data(), x.dim_size(0), y.dim_size(1),
                                        x.dim_size(1), 1.0f, static_cast<SM120DataType>(ToSM120<T>::value), stream);
      }
    }
    OP_REQUIRES(ctx, rc == cudaSuccess, errors::Internal("SM120 backward op failed: ", sm120_get_error_string(rc)));
  }
};

template <typename T>
class SM120FusedActivationOp : public OpKernel {
 public:
  explicit SM120FusedActivationOp(OpKernelConstruction* ctx) : OpKernel(ctx) {
    std::string name;
    OP_REQUIRES_OK(ctx, ctx->GetAttr("activation", &name));
    // the reference maps "gelu" to its tanh form here (src/tensorflow_ops/sm120_ops.cc:299) and unknown names to relu (:300)
    if (name == "gelu") activation_ = SM120_ACTIVATION_GELU;
    else activation_ = ActivationCode(name) == -2 ? SM120_ACTIVATION_RELU : ActivationCode(name);
  }

  void Compute(OpKernelContext* ctx) override {
    const Tensor& in = ctx->input(0);
    Tensor* out = nullptr;
    OP_REQUIRES_OK(ctx, ctx->allocate_output(0, in.shape(), &out));
    if (in.NumElements() == 0) return;
    const cudaError_t rc = sm120_launch_bias_activation(in.flat<T>().data(), nullptr, SM120_DTYPE_FLOAT32, out->flat<T>().data(), 1,
                                                        in.NumElements(), static_cast<SM120ActivationType>(activation_),
                                                        static_cast<SM120DataType>(ToSM120<T>::value), StreamOf(ctx));
    OP_REQUIRES(ctx, rc == cudaSuccess, errors::Internal("SM120FusedActivation failed: ", sm120_get_error_string(rc)));
  }

 private:
  int activation_ = SM120_ACTIVATION_RELU;
};

#define SM120_REGISTER(T)                                                                                              \
  REGISTER_KERNEL_BUILDER(Name("SM120MatMul").Device(DEVICE_GPU).TypeConstraint<T>("T"), SM120MatMulOp<T>);            \
  REGISTER_KERNEL_BUILDER(Name("SM120AdvancedMatMul").Device(DEVICE_GPU).TypeConstraint<T>("T"), SM120MatMulOp<T>);    \
  REGISTER_KERNEL_BUILDER(Name("SM120DenseFused").Device(DEVICE_GPU).TypeConstraint<T>("T"), SM120DenseFusedOp<T>);            \
  REGISTER_KERNEL_BUILDER(Name("SM120MatMulGradA").Device(DEVICE_GPU).TypeConstraint<T>("T"), SM120BackwardOp<T, 0>);          \
  REGISTER_KERNEL_BUILDER(Name("SM120MatMulGradB").Device(DEVICE_GPU).TypeConstraint<T>("T"), SM120BackwardOp<T, 1>);          \
  REGISTER_KERNEL_BUILDER(Name("SM120BiasGrad").Device(DEVICE_GPU).TypeConstraint<T>("T"), SM120BackwardOp<T, 2>);             \
  REGISTER_KERNEL_BUILDER(Name("SM120FusedActivation").Device(DEVICE_GPU).TypeConstraint<T>("T"), SM120FusedActivationOp<T>);
SM120_REGISTER(float)
SM120_REGISTER(Eigen::half)
SM120_REGISTER(bfloat16)
#undef SM120_REGISTER
REGISTER_KERNEL_BUILDER(Name("SM120MatMulFP8").Device(DEVICE_GPU), SM120MatMulOp<float8_e4m3fn>);

}  // namespace tensorflow

#endif  // SM120_HAVE_TENSORFLOW
