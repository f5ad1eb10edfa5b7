// Length-checked inference entry point for callers that hand over raw buffers (a C host, a trusted-execution shim).
//
// Version 1 of the ABI carries an ELEMENT COUNT beside every pointer and a layout record; every count is checked
// against the layout (with overflow-checked products) BEFORE any pointer is read or written, so an undersized buffer is
// refused instead of overrun. The older pointer-only entry point stays exported so that existing binaries still link,
// but it never touches its arguments and always fails closed. The computation itself is y = x W^T + b with
// W [out, in], x [batch, in], accumulated left to right in fp32 (a fixed order: the same bits on every host).
//
// Behaviour of scirust-runtime/src/enclave.rs (EnclaveLayout, safe_enclave_infer_v1, safe_enclave_infer).
#include <cstddef>
#include <cstdint>

namespace {
constexpr int32_t kOk = 0, kErrNull = 1, kErrLength = 2, kErrOverflow = 3, kErrVersion = 4, kErrFlag = 5, kErrLegacy = 6,
                  kErrAlias = 7;
constexpr uint32_t kAbiVersion = 1;

bool mul(size_t a, size_t b, size_t* out) { return !__builtin_mul_overflow(a, b, out); }

bool overlaps(const float* a, size_t na, const float* b, size_t nb) {
  const uintptr_t a0 = reinterpret_cast<uintptr_t>(a), a1 = a0 + na * sizeof(float);
  const uintptr_t b0 = reinterpret_cast<uintptr_t>(b), b1 = b0 + nb * sizeof(float);
  return na && nb && a0 < b1 && b0 < a1;
}
}  // namespace

extern "C" {

struct SbrtEnclaveLayout {
  size_t batch, in_features, out_features;
  uint8_t has_bias;  // a byte, not a bool: every bit pattern is a valid value at this boundary; only 0 and 1 are accepted
};

uint32_t sbrt_enclave_abi_version() { return kAbiVersion; }

int32_t sbrt_enclave_infer_v1(uint32_t abi_version, const float* weights, size_t weights_len, const float* input,
                              size_t input_len, float* output, size_t output_len, const float* bias, size_t bias_len,
                              SbrtEnclaveLayout dims) {
  if (abi_version != kAbiVersion) return kErrVersion;
  if (dims.has_bias > 1) return kErrFlag;
  size_t need_w, need_x, need_y;
  if (!mul(dims.out_features, dims.in_features, &need_w) || !mul(dims.batch, dims.in_features, &need_x) ||
      !mul(dims.batch, dims.out_features, &need_y))
    return kErrOverflow;
  const size_t need_b = dims.has_bias ? dims.out_features : 0;
  if (weights_len != need_w || input_len != need_x || output_len != need_y || bias_len != need_b) return kErrLength;
  if ((need_w && !weights) || (need_x && !input) || (need_y && !output) || (need_b && !bias)) return kErrNull;
  if (!dims.has_bias && bias) return kErrFlag;
  if (overlaps(output, need_y, weights, need_w) || overlaps(output, need_y, input, need_x) ||
      overlaps(output, need_y, bias, need_b))
    return kErrAlias;
  for (size_t b = 0; b < dims.batch; ++b)
    for (size_t o = 0; o < dims.out_features; ++o) {
      float acc = dims.has_bias ? bias[o] : 0.0f;
      const float* w = weights + o * dims.in_features;
      const float* x = input + b * dims.in_features;
      for (size_t i = 0; i < dims.in_features; ++i) acc += w[i] * x[i];
      output[b * dims.out_features + o] = acc;
    }
  return kOk;
}

// Pointer-only predecessor: cannot know any buffer's size, so it reads nothing and refuses.
int32_t sbrt_enclave_infer(const float*, const float*, float*, const float*, SbrtEnclaveLayout) { return kErrLegacy; }

}  // extern "C"
