// torch stable-ABI operators of namespace consumer_int8 for the W8A8 linear path, as thin
// wrappers over the C ABI in include/ci8.h. Schemas, argument checks and error texts follow the
// reference's csrc/bindings.cpp (quantize_rows :191-209, quantize_grouped4096 :210-237,
// channel_mm :238-265, channel_gemv :289-310, cutlass/fused_channel_mm :386-427, schemas
// :593-613). Every output is caller-owned; nothing here allocates or synchronises.
#include <Python.h>
#include <torch/csrc/stable/library.h>
#include <torch/csrc/stable/tensor.h>
#include <torch/csrc/stable/accelerator.h>
#include <torch/csrc/inductor/aoti_torch/c/shim.h>
#include <torch/headeronly/util/Exception.h>
#include <cstdint>
#include <limits>
#include "../../include/ci8.h"

using torch::stable::Tensor;
using torch::headeronly::ScalarType;

namespace {
using torch::stable::detail::to;
constexpr int64_t kIntMax = std::numeric_limits<int>::max();

void check(const Tensor& t, ScalarType dtype, int device) {
  STD_TORCH_CHECK(t.is_cuda() && t.get_device_index() == device,
                  "All tensors must be on the same CUDA device");
  STD_TORCH_CHECK(t.is_contiguous() && t.scalar_type() == dtype,
                  "Unexpected dtype or noncontiguous tensor");
}
ci8_stream_t stream_for(int device) {
  void* stream = nullptr;
  TORCH_ERROR_CODE_CHECK(aoti_torch_get_current_cuda_stream(device, &stream));
  return reinterpret_cast<ci8_stream_t>(stream);
}
void launched(int code) { STD_TORCH_CHECK(code == 0, ci8_error_string(code)); }
uintptr_t address(const Tensor& t) { return reinterpret_cast<uintptr_t>(t.data_ptr()); }

void boxed_quant(StableIValue* stack, uint64_t, uint64_t) {
  auto x = to<Tensor>(stack[0]), codes = to<Tensor>(stack[1]), scale = to<Tensor>(stack[2]);
  const int device = x.get_device_index();
  check(x, ScalarType::BFloat16, device);
  check(codes, ScalarType::Char, device);
  check(scale, ScalarType::Float, device);
  STD_TORCH_CHECK(x.dim() == 2 && x.size(0) > 0 && x.size(1) > 0, "Expected a nonempty BF16 matrix");
  STD_TORCH_CHECK(codes.dim() == 2 && codes.size(0) == x.size(0) && codes.size(1) == x.size(1) &&
                      scale.dim() == 1 && scale.size(0) == x.size(0),
                  "Wrong output shapes");
  STD_TORCH_CHECK(x.numel() <= kIntMax, "Matrix too large");
  torch::stable::accelerator::DeviceGuard guard(device);
  launched(ci8_quantize_rows(x.data_ptr(), static_cast<int8_t*>(codes.data_ptr()),
                             static_cast<float*>(scale.data_ptr()), x.size(0), x.size(1),
                             stream_for(device)));
}

// silu_mul / silu_mul_quantize: reference csrc/bindings.cpp:32-65 (any width % 8 == 0 is accepted
// here; the reference takes 8704 and 17408 only).
void boxed_silu_mul(StableIValue* stack, uint64_t, uint64_t) {
  auto x = to<Tensor>(stack[0]), out = to<Tensor>(stack[1]);
  const int device = x.get_device_index();
  check(x, ScalarType::BFloat16, device);
  check(out, ScalarType::BFloat16, device);
  STD_TORCH_CHECK(x.dim() == 2 && out.dim() == 2 && out.size(1) > 0 && out.size(1) % 8 == 0 &&
                      x.size(1) == 2 * out.size(1) && x.size(0) == out.size(0) && x.numel() <= kIntMax,
                  "Unsupported SwiGLU shape");
  STD_TORCH_CHECK(address(x) % 16 == 0 && address(out) % 16 == 0, "SwiGLU requires aligned buffers");
  torch::stable::accelerator::DeviceGuard guard(device);
  launched(ci8_silu_mul(x.data_ptr(), out.data_ptr(), x.size(0), out.size(1), stream_for(device)));
}

void boxed_silu_quant(StableIValue* stack, uint64_t, uint64_t) {
  auto x = to<Tensor>(stack[0]), codes = to<Tensor>(stack[1]), scales = to<Tensor>(stack[2]);
  const int device = x.get_device_index();
  check(x, ScalarType::BFloat16, device);
  check(codes, ScalarType::Char, device);
  check(scales, ScalarType::Float, device);
  STD_TORCH_CHECK(x.dim() == 2 && codes.dim() == 2 && scales.dim() == 1 && codes.size(1) > 0 &&
                      codes.size(1) % 8 == 0 && codes.size(1) <= 65536 && x.size(1) == 2 * codes.size(1) &&
                      x.size(0) == codes.size(0) && scales.size(0) == x.size(0) && x.numel() <= kIntMax,
                  "Unsupported SwiGLU quantization shape");
  STD_TORCH_CHECK(address(x) % 16 == 0 && address(codes) % 8 == 0, "SwiGLU quantization requires aligned buffers");
  torch::stable::accelerator::DeviceGuard guard(device);
  launched(ci8_silu_mul_quantize(x.data_ptr(), static_cast<int8_t*>(codes.data_ptr()),
                                 static_cast<float*>(scales.data_ptr()), x.size(0), codes.size(1),
                                 stream_for(device)));
}

void boxed_grouped_quant(StableIValue* stack, uint64_t, uint64_t) {
  auto x = to<Tensor>(stack[0]), codes = to<Tensor>(stack[1]), scales = to<Tensor>(stack[2]);
  const int device = x.get_device_index();
  check(x, ScalarType::BFloat16, device);
  check(codes, ScalarType::Char, device);
  check(scales, ScalarType::Float, device);
  STD_TORCH_CHECK(x.dim() == 3 && x.size(1) > 0 && x.size(2) == 4096 && codes.dim() == 3 &&
                      codes.size(0) == x.size(1) && codes.size(1) == x.size(0) && codes.size(2) == 4096 &&
                      scales.dim() == 2 && scales.size(0) == x.size(1) && scales.size(1) == x.size(0) &&
                      x.numel() <= kIntMax,
                  "Expected BF16 input[M,G,4096], INT8 codes[G,M,4096], FP32 scales[G,M]");
  STD_TORCH_CHECK(address(x) % 16 == 0 && address(codes) % 8 == 0 && address(scales) % 4 == 0,
                  "Grouped quantization requires aligned buffers");
  auto overlap = [](const Tensor& a, int64_t bytes_a, const Tensor& b, int64_t bytes_b) {
    const uintptr_t first = address(a), second = address(b);
    return a.numel() && b.numel() && first < second + b.numel() * bytes_b &&
           second < first + a.numel() * bytes_a;
  };
  STD_TORCH_CHECK(!overlap(x, 2, codes, 1) && !overlap(x, 2, scales, 4) && !overlap(codes, 1, scales, 4),
                  "Grouped quantization buffers must not overlap");
  torch::stable::accelerator::DeviceGuard guard(device);
  launched(ci8_quantize_grouped4096(x.data_ptr(), static_cast<int8_t*>(codes.data_ptr()),
                                    static_cast<float*>(scales.data_ptr()), x.size(0), x.size(1),
                                    stream_for(device)));
}

void boxed_mm(StableIValue* stack, uint64_t, uint64_t) {
  auto a = to<Tensor>(stack[0]), w = to<Tensor>(stack[1]), sa = to<Tensor>(stack[2]);
  auto sw = to<Tensor>(stack[3]), out = to<Tensor>(stack[4]);
  const int device = a.get_device_index();
  check(a, ScalarType::Char, device);
  check(w, ScalarType::Byte, device);
  check(sa, ScalarType::Float, device);
  check(sw, ScalarType::BFloat16, device);
  check(out, ScalarType::BFloat16, device);
  STD_TORCH_CHECK(a.dim() == 2 && w.dim() == 2 && out.dim() == 2, "Expected matrices");
  const int64_t m = a.size(0), n = w.size(0), k = a.size(1);
  STD_TORCH_CHECK(m > 0 && n > 0 && k > 0 && k % 32 == 0 && k <= 65536 && w.size(1) == k,
                  "Invalid matrix geometry");
  STD_TORCH_CHECK(sa.dim() == 1 && sa.size(0) == m && sw.dim() == 1 && sw.size(0) == n &&
                      out.size(0) == m && out.size(1) == n,
                  "Wrong scale or output shapes");
  STD_TORCH_CHECK(a.numel() <= kIntMax && w.numel() <= kIntMax, "Matrix too large");
  // the reference reads both operands as 32-bit words and asks for nothing more; operands that are
  // not 16-byte aligned take the library's plain word-wise kernel instead of the TMA paths
  STD_TORCH_CHECK(address(a) % 4 == 0 && address(w) % 4 == 0, "Matrix operands must be 4-byte aligned");
  torch::stable::accelerator::DeviceGuard guard(device);
  launched(ci8_channel_mm(static_cast<int8_t*>(a.data_ptr()), static_cast<uint8_t*>(w.data_ptr()),
                          static_cast<float*>(sa.data_ptr()), sw.data_ptr(), out.data_ptr(), m, n, k,
                          stream_for(device)));
}

// unpack_allspark: reference csrc/bindings.cpp:266-288.
void boxed_unpack_allspark(StableIValue* stack, uint64_t, uint64_t) {
  auto packed = to<Tensor>(stack[0]), packed_scales = to<Tensor>(stack[1]);
  auto weight = to<Tensor>(stack[2]), scales = to<Tensor>(stack[3]);
  const int device = packed.get_device_index();
  check(packed, ScalarType::Byte, device);
  check(packed_scales, ScalarType::BFloat16, device);
  check(weight, ScalarType::Char, device);
  check(scales, ScalarType::BFloat16, device);
  STD_TORCH_CHECK(packed.dim() == 2 && weight.dim() == 2 && packed_scales.dim() == 1 && scales.dim() == 1,
                  "Wrong tensor ranks");
  const int64_t n = weight.size(0), k = weight.size(1), padded_n = (n + 31) / 32 * 32;
  STD_TORCH_CHECK(n > 0 && n % 16 == 0 && k > 0 && k <= 65536 && k % 16 == 0 && packed.size(0) == padded_n &&
                      packed.size(1) == k && packed_scales.size(0) == padded_n && scales.size(0) == n,
                  "Expected AllSpark N32K16 weights and channel scales");
  STD_TORCH_CHECK(packed.numel() <= kIntMax, "Weight too large");
  STD_TORCH_CHECK(address(packed) % 16 == 0 && address(weight) % 16 == 0, "Unaligned weights");
  torch::stable::accelerator::DeviceGuard guard(device);
  launched(ci8_unpack_allspark(static_cast<uint8_t*>(packed.data_ptr()), packed_scales.data_ptr(),
                               static_cast<int8_t*>(weight.data_ptr()), scales.data_ptr(), n, k,
                               stream_for(device)));
}

void boxed_gemv(StableIValue* stack, uint64_t, uint64_t) {
  auto x = to<Tensor>(stack[0]), w = to<Tensor>(stack[1]);
  auto scale = to<Tensor>(stack[2]), out = to<Tensor>(stack[3]);
  const int device = x.get_device_index();
  check(x, ScalarType::BFloat16, device);
  check(w, ScalarType::Char, device);
  check(scale, ScalarType::BFloat16, device);
  check(out, ScalarType::BFloat16, device);
  STD_TORCH_CHECK(x.dim() == 2 && w.dim() == 2 && out.dim() == 2 && scale.dim() == 1,
                  "Expected input/weight/output matrices and channel scales");
  const int64_t m = x.size(0), n = w.size(0), k = x.size(1);
  // The reference stops at 8 rows; this build accepts up to 16 (a superset).
  STD_TORCH_CHECK(m > 0 && m <= 16 && n > 0 && k > 0 && k <= 65536 && k % 16 == 0 && w.size(1) == k &&
                      scale.size(0) == n && out.size(0) == m && out.size(1) == n,
                  "Unsupported W8A16 GEMV geometry");
  STD_TORCH_CHECK(w.numel() <= kIntMax, "Weight matrix too large");
  STD_TORCH_CHECK(address(w) % 16 == 0 && address(x) % 4 == 0, "Unaligned vector inputs");
  torch::stable::accelerator::DeviceGuard guard(device);
  launched(ci8_channel_gemv(x.data_ptr(), static_cast<int8_t*>(w.data_ptr()), scale.data_ptr(),
                            out.data_ptr(), m, n, k, stream_for(device)));
}

void tiled_mm_impl(StableIValue* stack, bool fused) {
  auto a = to<Tensor>(stack[0]), w = to<Tensor>(stack[1]);
  auto sa = to<Tensor>(stack[2]), sw = to<Tensor>(stack[3]);
  auto out = to<Tensor>(stack[fused ? 4 : 5]);
  const int device = a.get_device_index();
  check(a, ScalarType::Char, device);
  check(w, ScalarType::Char, device);
  check(sa, ScalarType::Float, device);
  check(sw, ScalarType::BFloat16, device);
  check(out, ScalarType::BFloat16, device);
  STD_TORCH_CHECK(a.dim() == 2 && w.dim() == 2 && out.dim() == 2, "Expected matrices");
  const int64_t m = a.size(0), n = w.size(0), k = a.size(1);
  STD_TORCH_CHECK(m > 0 && n > 0 && k > 0 && n % 4 == 0 && k % 32 == 0 && k <= 65536 && w.size(1) == k &&
                      out.size(0) == m && out.size(1) == n && sa.dim() == 1 && sw.dim() == 1 &&
                      sa.size(0) == m && sw.size(0) == n,
                  "Invalid CUTLASS geometry");
  STD_TORCH_CHECK(a.numel() <= kIntMax && w.numel() <= kIntMax && out.numel() <= kIntMax, "Matrix too large");
  STD_TORCH_CHECK(address(a) % 16 == 0 && address(w) % 16 == 0, "Matrix operands must be 16-byte aligned");
  torch::stable::accelerator::DeviceGuard guard(device);
  if (fused) {
    const int64_t schedule = to<int64_t>(stack[5]);
    STD_TORCH_CHECK(schedule >= 0 && schedule <= 6, "Invalid fused GEMM schedule");
    launched(ci8_fused_channel_mm(static_cast<int8_t*>(a.data_ptr()), static_cast<int8_t*>(w.data_ptr()),
                                  static_cast<float*>(sa.data_ptr()), sw.data_ptr(), out.data_ptr(), m, n, k,
                                  static_cast<int>(schedule), stream_for(device)));
  } else {
    auto workspace = to<Tensor>(stack[4]);
    check(workspace, ScalarType::Int, device);
    STD_TORCH_CHECK(workspace.dim() == 2 && workspace.size(0) == m && workspace.size(1) == n,
                    "Expected matching workspace");
    launched(ci8_cutlass_channel_mm(static_cast<int8_t*>(a.data_ptr()), static_cast<int8_t*>(w.data_ptr()),
                                    static_cast<float*>(sa.data_ptr()), sw.data_ptr(),
                                    static_cast<int32_t*>(workspace.data_ptr()), out.data_ptr(), m, n, k,
                                    stream_for(device)));
  }
}
void boxed_cutlass_mm(StableIValue* stack, uint64_t, uint64_t) { tiled_mm_impl(stack, false); }
void boxed_fused_mm(StableIValue* stack, uint64_t, uint64_t) { tiled_mm_impl(stack, true); }

// Additive operator (no counterpart in the reference's surface): the grouped-scale GEMM in one
// launch, consuming what quantize_grouped4096 writes.
// The _ws form takes a caller-lent BYTE workspace (zero before its first use) in front of `out`; with
// at least ci8_grouped_workspace_bytes() of it the tiles of a thin last wave are split along the groups.
void grouped_mm_impl(StableIValue* stack, bool with_workspace) {
  auto codes = to<Tensor>(stack[0]), w = to<Tensor>(stack[1]), scales = to<Tensor>(stack[2]);
  auto sw = to<Tensor>(stack[3]), out = to<Tensor>(stack[with_workspace ? 5 : 4]);
  const int device = codes.get_device_index();
  check(codes, ScalarType::Char, device);
  check(w, ScalarType::Char, device);
  check(scales, ScalarType::Float, device);
  check(sw, ScalarType::BFloat16, device);
  check(out, ScalarType::BFloat16, device);
  STD_TORCH_CHECK(codes.dim() == 3 && codes.size(2) == 4096 && w.dim() == 2 && scales.dim() == 2 &&
                      sw.dim() == 1 && out.dim() == 2,
                  "Expected INT8 codes[G,M,4096], INT8 w[N,G*4096], FP32 scales[G,M], BF16 w_scale[N], BF16 out[M,N]");
  const int64_t groups = codes.size(0), m = codes.size(1), n = w.size(0);
  STD_TORCH_CHECK(groups > 0 && groups <= 16 && m > 0 && n > 0 && w.size(1) == groups * 4096 &&
                      scales.size(0) == groups && scales.size(1) == m && sw.size(0) == n &&
                      out.size(0) == m && out.size(1) == n,
                  "Invalid grouped GEMM geometry");
  STD_TORCH_CHECK(codes.numel() <= kIntMax && w.numel() <= kIntMax && out.numel() <= kIntMax, "Matrix too large");
  STD_TORCH_CHECK(address(codes) % 16 == 0 && address(w) % 16 == 0, "Matrix operands must be 16-byte aligned");
  void* workspace = nullptr;
  long long workspace_bytes = 0;
  if (with_workspace) {
    auto lent = to<Tensor>(stack[4]);
    check(lent, ScalarType::Byte, device);
    STD_TORCH_CHECK(address(lent) % 16 == 0, "The workspace must be 16-byte aligned");
    workspace = lent.data_ptr();
    workspace_bytes = lent.numel();
  }
  torch::stable::accelerator::DeviceGuard guard(device);
  launched(ci8_grouped_channel_mm_ws(static_cast<int8_t*>(codes.data_ptr()), static_cast<int8_t*>(w.data_ptr()),
                                     static_cast<float*>(scales.data_ptr()), sw.data_ptr(), out.data_ptr(), workspace,
                                     workspace_bytes, m, n, groups, stream_for(device)));
}
void boxed_grouped_mm(StableIValue* stack, uint64_t, uint64_t) { grouped_mm_impl(stack, false); }
void boxed_grouped_mm_ws(StableIValue* stack, uint64_t, uint64_t) { grouped_mm_impl(stack, true); }

// Additive operator: quantize_rows + fused_channel_mm as one call (one kernel for decode shapes); codes and
// scales receive what quantize_rows would write.
void boxed_dynamic_mm(StableIValue* stack, uint64_t, uint64_t) {
  auto x = to<Tensor>(stack[0]), w = to<Tensor>(stack[1]), sw = to<Tensor>(stack[2]);
  auto codes = to<Tensor>(stack[3]), scales = to<Tensor>(stack[4]), out = to<Tensor>(stack[5]);
  const int device = x.get_device_index();
  check(x, ScalarType::BFloat16, device);
  check(w, ScalarType::Char, device);
  check(sw, ScalarType::BFloat16, device);
  check(codes, ScalarType::Char, device);
  check(scales, ScalarType::Float, device);
  check(out, ScalarType::BFloat16, device);
  STD_TORCH_CHECK(x.dim() == 2 && w.dim() == 2 && sw.dim() == 1 && codes.dim() == 2 && scales.dim() == 1 && out.dim() == 2,
                  "Expected BF16 x[M,K], INT8 w[N,K], BF16 w_scale[N], INT8 codes[M,K], FP32 scales[M], BF16 out[M,N]");
  const int64_t m = x.size(0), k = x.size(1), n = w.size(0);
  STD_TORCH_CHECK(m > 0 && n > 0 && n % 4 == 0 && k > 0 && k % 32 == 0 && k <= 65536 && w.size(1) == k &&
                      sw.size(0) == n && codes.size(0) == m && codes.size(1) == k && scales.size(0) == m &&
                      out.size(0) == m && out.size(1) == n,
                  "Invalid dynamic GEMM geometry");
  STD_TORCH_CHECK(x.numel() <= kIntMax && w.numel() <= kIntMax && out.numel() <= kIntMax, "Matrix too large");
  STD_TORCH_CHECK(address(x) % 16 == 0 && address(w) % 16 == 0 && address(codes) % 16 == 0,
                  "Matrix operands must be 16-byte aligned");
  torch::stable::accelerator::DeviceGuard guard(device);
  launched(ci8_dynamic_channel_mm(x.data_ptr(), static_cast<int8_t*>(w.data_ptr()), sw.data_ptr(),
                                  static_cast<int8_t*>(codes.data_ptr()), static_cast<float*>(scales.data_ptr()),
                                  out.data_ptr(), m, n, k, stream_for(device)));
}

// Additive operator: gate/up projection with the SwiGLU in the GEMM epilogue; the same bits as
// fused_channel_mm followed by silu_mul. w / w_scale rows are gate and up interleaved in blocks of 128.
void boxed_gate_up_silu_mm(StableIValue* stack, uint64_t, uint64_t) {
  auto a = to<Tensor>(stack[0]), w = to<Tensor>(stack[1]), sa = to<Tensor>(stack[2]);
  auto sw = to<Tensor>(stack[3]), out = to<Tensor>(stack[4]);
  const int device = a.get_device_index();
  check(a, ScalarType::Char, device);
  check(w, ScalarType::Char, device);
  check(sa, ScalarType::Float, device);
  check(sw, ScalarType::BFloat16, device);
  check(out, ScalarType::BFloat16, device);
  STD_TORCH_CHECK(a.dim() == 2 && w.dim() == 2 && sa.dim() == 1 && sw.dim() == 1 && out.dim() == 2,
                  "Expected INT8 a[M,K], INT8 w[N,K], FP32 a_scale[M], BF16 w_scale[N], BF16 out[M,N/2]");
  const int64_t m = a.size(0), k = a.size(1), n = w.size(0);
  STD_TORCH_CHECK(m > 0 && n > 0 && n % 256 == 0 && k > 0 && k % 32 == 0 && k <= 65536 && w.size(1) == k &&
                      sa.size(0) == m && sw.size(0) == n && out.size(0) == m && out.size(1) == n / 2,
                  "Invalid gate/up GEMM geometry");
  STD_TORCH_CHECK(a.numel() <= kIntMax && w.numel() <= kIntMax && m * n <= kIntMax, "Matrix too large");
  STD_TORCH_CHECK(address(a) % 16 == 0 && address(w) % 16 == 0 && address(out) % 16 == 0,
                  "Matrix operands must be 16-byte aligned");
  torch::stable::accelerator::DeviceGuard guard(device);
  launched(ci8_gate_up_silu_mm(static_cast<int8_t*>(a.data_ptr()), static_cast<int8_t*>(w.data_ptr()),
                               static_cast<float*>(sa.data_ptr()), sw.data_ptr(), out.data_ptr(), m, n, k,
                               stream_for(device)));
}

// Additive operators: this rank's output-channel shard of fused_channel_mm, written straight into
// block `rank` of every rank's gathered buffer [world, M, N/world] (peer-mapped symmetric memory).
// peer_ptrs is a CPU INT64 tensor holding the device address of every rank's buffer. The _sync form
// also takes signal_ptrs (CPU INT64, the address of every rank's arrival counters) and state (INT64
// [4] on this device) and ends with the in-kernel cross-GPU rendezvous.
void gather_common(StableIValue* stack, bool sync) {
  auto a = to<Tensor>(stack[0]), w = to<Tensor>(stack[1]);
  auto sa = to<Tensor>(stack[2]), sw = to<Tensor>(stack[3]);
  auto gathered = to<Tensor>(stack[4]), peer_ptrs = to<Tensor>(stack[5]);
  const int base = sync ? 8 : 6;
  const int64_t rank = to<int64_t>(stack[base]), schedule = to<int64_t>(stack[base + 1]);
  const int device = a.get_device_index();
  check(a, ScalarType::Char, device);
  check(w, ScalarType::Char, device);
  check(sa, ScalarType::Float, device);
  check(sw, ScalarType::BFloat16, device);
  check(gathered, ScalarType::BFloat16, device);
  STD_TORCH_CHECK(!peer_ptrs.is_cuda() && peer_ptrs.is_contiguous() && peer_ptrs.scalar_type() == ScalarType::Long &&
                      peer_ptrs.dim() == 1,
                  "peer_ptrs must be a contiguous CPU INT64 vector");
  STD_TORCH_CHECK(a.dim() == 2 && w.dim() == 2 && gathered.dim() == 3, "Expected matrices and a [world,M,N/world] buffer");
  const int64_t m = a.size(0), n = w.size(0), k = a.size(1), world = peer_ptrs.size(0);
  STD_TORCH_CHECK(m > 0 && n > 0 && k > 0 && n % 8 == 0 && k % 32 == 0 && k <= 65536 && w.size(1) == k &&
                      world > 0 && world <= 8 && rank >= 0 && rank < world && gathered.size(0) == world &&
                      gathered.size(1) == m && gathered.size(2) == n && sa.dim() == 1 && sw.dim() == 1 &&
                      sa.size(0) == m && sw.size(0) == n,
                  "Invalid sharded GEMM geometry");
  STD_TORCH_CHECK(a.numel() <= kIntMax && w.numel() <= kIntMax && gathered.numel() <= kIntMax, "Matrix too large");
  STD_TORCH_CHECK(schedule >= 0 && schedule <= 6, "Invalid fused GEMM schedule");
  const int64_t* addresses = static_cast<const int64_t*>(peer_ptrs.data_ptr());
  STD_TORCH_CHECK(static_cast<uintptr_t>(addresses[rank]) == address(gathered),
                  "peer_ptrs[rank] must be the address of this rank's gathered buffer");
  void* buffers[8];
  for (int64_t r = 0; r < world; ++r) buffers[r] = reinterpret_cast<void*>(static_cast<uintptr_t>(addresses[r]));
  STD_TORCH_CHECK(address(a) % 16 == 0 && address(w) % 16 == 0, "Matrix operands must be 16-byte aligned");
  if (!sync) {
    torch::stable::accelerator::DeviceGuard guard(device);
    launched(ci8_fused_channel_mm_gather(static_cast<int8_t*>(a.data_ptr()), static_cast<int8_t*>(w.data_ptr()),
                                         static_cast<float*>(sa.data_ptr()), sw.data_ptr(), buffers,
                                         static_cast<int>(world), static_cast<int>(rank), m, n, k,
                                         static_cast<int>(schedule), stream_for(device)));
    return;
  }
  auto signal_ptrs = to<Tensor>(stack[6]), state = to<Tensor>(stack[7]);
  check(state, ScalarType::Long, device);
  STD_TORCH_CHECK(state.numel() == 4, "state must hold four INT64 words");
  STD_TORCH_CHECK(!signal_ptrs.is_cuda() && signal_ptrs.is_contiguous() && signal_ptrs.scalar_type() == ScalarType::Long &&
                      signal_ptrs.dim() == 1 && signal_ptrs.size(0) == world,
                  "signal_ptrs must be a contiguous CPU INT64 vector with one entry per rank");
  const int64_t* signal_addresses = static_cast<const int64_t*>(signal_ptrs.data_ptr());
  void* signals[8];
  for (int64_t r = 0; r < world; ++r) signals[r] = reinterpret_cast<void*>(static_cast<uintptr_t>(signal_addresses[r]));
  torch::stable::accelerator::DeviceGuard guard(device);
  launched(ci8_fused_channel_mm_gather_sync(static_cast<int8_t*>(a.data_ptr()), static_cast<int8_t*>(w.data_ptr()),
                                            static_cast<float*>(sa.data_ptr()), sw.data_ptr(), buffers, signals,
                                            state.data_ptr(), static_cast<int>(world), static_cast<int>(rank), m, n, k,
                                            static_cast<int>(schedule), stream_for(device)));
}
// peer_rendezvous(signal_ptrs CPU INT64[world], state INT64[2] on this device, rank): the closing barrier
// of fused_channel_mm_gather as a kernel of its own.
void boxed_peer_rendezvous(StableIValue* stack, uint64_t, uint64_t) {
  auto signal_ptrs = to<Tensor>(stack[0]), state = to<Tensor>(stack[1]);
  const int64_t rank = to<int64_t>(stack[2]);
  const int device = state.get_device_index();
  check(state, ScalarType::Long, device);
  STD_TORCH_CHECK(state.numel() == 2 || state.numel() == 4, "state must hold two (or the gathering operator's four) INT64 words");
  STD_TORCH_CHECK(!signal_ptrs.is_cuda() && signal_ptrs.is_contiguous() && signal_ptrs.scalar_type() == ScalarType::Long &&
                      signal_ptrs.dim() == 1 && signal_ptrs.size(0) > 0 && signal_ptrs.size(0) <= 8,
                  "signal_ptrs must be a contiguous CPU INT64 vector with one entry per rank");
  const int64_t world = signal_ptrs.size(0);
  STD_TORCH_CHECK(rank >= 0 && rank < world, "rank outside the world");
  const int64_t* addresses = static_cast<const int64_t*>(signal_ptrs.data_ptr());
  void* signals[8];
  for (int64_t r = 0; r < world; ++r) signals[r] = reinterpret_cast<void*>(static_cast<uintptr_t>(addresses[r]));
  torch::stable::accelerator::DeviceGuard guard(device);
  launched(ci8_peer_rendezvous(signals, state.data_ptr(), static_cast<int>(world), static_cast<int>(rank),
                               stream_for(device)));
}
void boxed_fused_mm_gather(StableIValue* stack, uint64_t, uint64_t) { gather_common(stack, false); }
void boxed_fused_mm_gather_sync(StableIValue* stack, uint64_t, uint64_t) { gather_common(stack, true); }
}  // namespace

STABLE_TORCH_LIBRARY(consumer_int8, m) {
  m.def("silu_mul(Tensor input, Tensor(a!) out) -> ()");
  m.def("silu_mul_quantize(Tensor input, Tensor(a!) codes, Tensor(b!) scales) -> ()");
  m.def("fused_channel_mm(Tensor a, Tensor w, Tensor a_scale, Tensor w_scale, Tensor(a!) out, int schedule=0) -> ()");
  m.def("quantize_rows(Tensor input, Tensor(a!) codes, Tensor(b!) scales) -> ()");
  m.def("quantize_grouped4096(Tensor input, Tensor(a!) codes, Tensor(b!) scales) -> ()");
  m.def("channel_mm(Tensor a, Tensor w, Tensor a_scale, Tensor w_scale, Tensor(a!) out) -> ()");
  m.def("unpack_allspark(Tensor packed, Tensor packed_scales, Tensor(a!) weight, Tensor(b!) scales) -> ()");
  m.def("channel_gemv(Tensor x, Tensor w, Tensor scale, Tensor(a!) out) -> ()");
  m.def("cutlass_channel_mm(Tensor a, Tensor w, Tensor a_scale, Tensor w_scale, Tensor(a!) workspace, Tensor(b!) out) -> ()");
  m.def("grouped_channel_mm(Tensor codes, Tensor w, Tensor scales, Tensor w_scale, Tensor(a!) out) -> ()");
  m.def("grouped_channel_mm_ws(Tensor codes, Tensor w, Tensor scales, Tensor w_scale, Tensor(a!) workspace, Tensor(b!) out) -> ()");
  m.def("dynamic_channel_mm(Tensor x, Tensor w, Tensor w_scale, Tensor(a!) codes, Tensor(b!) scales, Tensor(c!) out) -> ()");
  m.def("gate_up_silu_mm(Tensor a, Tensor w, Tensor a_scale, Tensor w_scale, Tensor(a!) out) -> ()");
  m.def("fused_channel_mm_gather(Tensor a, Tensor w, Tensor a_scale, Tensor w_scale, Tensor(a!) gathered, Tensor peer_ptrs, int rank, int schedule=0) -> ()");
  m.def("peer_rendezvous(Tensor signal_ptrs, Tensor(a!) state, int rank) -> ()");
  m.def("fused_channel_mm_gather_sync(Tensor a, Tensor w, Tensor a_scale, Tensor w_scale, Tensor(a!) gathered, Tensor peer_ptrs, Tensor signal_ptrs, Tensor(b!) state, int rank, int schedule=0) -> ()");
}
STABLE_TORCH_LIBRARY_IMPL(consumer_int8, CUDA, m) {
  m.impl("silu_mul", &boxed_silu_mul);
  m.impl("silu_mul_quantize", &boxed_silu_quant);
  m.impl("fused_channel_mm", &boxed_fused_mm);
  m.impl("quantize_rows", &boxed_quant);
  m.impl("quantize_grouped4096", &boxed_grouped_quant);
  m.impl("channel_mm", &boxed_mm);
  m.impl("unpack_allspark", &boxed_unpack_allspark);
  m.impl("channel_gemv", &boxed_gemv);
  m.impl("cutlass_channel_mm", &boxed_cutlass_mm);
  m.impl("grouped_channel_mm", &boxed_grouped_mm);
  m.impl("grouped_channel_mm_ws", &boxed_grouped_mm_ws);
  m.impl("gate_up_silu_mm", &boxed_gate_up_silu_mm);
  m.impl("dynamic_channel_mm", &boxed_dynamic_mm);
  m.impl("fused_channel_mm_gather", &boxed_fused_mm_gather);
  m.impl("fused_channel_mm_gather_sync", &boxed_fused_mm_gather_sync);
  m.impl("peer_rendezvous", &boxed_peer_rendezvous);
}
extern "C" PyObject* PyInit__C() {
  static PyModuleDef module = {PyModuleDef_HEAD_INIT, "_C", nullptr, -1, nullptr};
  return PyModule_Create(&module);
}
