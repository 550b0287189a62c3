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
// Differences from the reference glue, all deliberate: the shape function
// honours the transposes (the reference's ignores them, :91-99); an unsupported
// dtype is an error instead of silently becoming FLOAT32 (:44-53); T also
// admits bfloat16.
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

    SM120GemmDesc d;
    sm120_gemm_desc_init(&d);
    d.A = a.flat<T>().data();
    d.B = b.flat<T>().data();
    d.C = out->flat<T>().data();
    d.M = a_rows; d.N = b_cols; d.K = a_cols;
    d.transpose_a = transpose_a_; d.transpose_b = transpose_b_;
    d.in_dtype = d.out_dtype = ToSM120<T>::value;
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

#define SM120_REGISTER(T)                                                                                              \
  REGISTER_KERNEL_BUILDER(Name("SM120MatMul").Device(DEVICE_GPU).TypeConstraint<T>("T"), SM120MatMulOp<T>);            \
  REGISTER_KERNEL_BUILDER(Name("SM120AdvancedMatMul").Device(DEVICE_GPU).TypeConstraint<T>("T"), SM120MatMulOp<T>);    \
  REGISTER_KERNEL_BUILDER(Name("SM120DenseFused").Device(DEVICE_GPU).TypeConstraint<T>("T"), SM120DenseFusedOp<T>);
SM120_REGISTER(float)
SM120_REGISTER(Eigen::half)
SM120_REGISTER(bfloat16)
#undef SM120_REGISTER

}  // namespace tensorflow

#endif  // SM120_HAVE_TENSORFLOW
