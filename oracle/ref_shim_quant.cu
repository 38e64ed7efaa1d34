// C-ABI shim around the reference's quantizer kernels (eiz/llama.cu, transform.cu:28-150).
//
// TEST INFRASTRUCTURE ONLY.  transform.cu is a program with its own main(); it is included from
// where it lies with main renamed, so that its kernels can be launched on caller-provided data
// with exactly the launch shapes its quantize_one() uses (transform.cu:171-175).
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <string>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#define main ref_transform_main
#include "transform.cu"
#undef main

using namespace llama_cu;

extern "C" {

// fp16 (h,w) host matrix -> u8 values + fp16 scales, block size bs along w.  Also returns the
// reference's round-trip statistics (mean squared, max, mean absolute error) in stats[3].
int ref_quantize_absmax_uint8(uint8_t* q_out, uint16_t* scales_out, const uint16_t* in, uint64_t h, uint64_t w, int bs,
                              float* stats) {
  tensor4d<half> input(1, 1, h, w), scales(1, 1, h, w / bs), deq(1, 1, h, w);
  tensor4d<uint8_t> output(1, 1, h, w);
  tensor4d<float> error(1, 1, 1, 3);
  cudaMemcpy(input.data(), in, h * w * 2, cudaMemcpyHostToDevice);
  cudaMemset(error.data(), 0, 12);
  quantize_absmax_uint8<<<dim3(w / bs, h), std::min(bs, 1024)>>>(output.data(), scales.data(), input.data(), h, w, bs);
  dequantize_absmax_uint8<<<dim3(w / bs, h), std::min(bs, 1024)>>>(deq.data(), scales.data(), output.data(), h, w, bs);
  error_stats<<<128, 1024>>>(error.data(), input.data(), deq.data(), h * w);
  if (cudaDeviceSynchronize() != cudaSuccess) return 1;
  cudaMemcpy(q_out, output.data(), h * w, cudaMemcpyDeviceToHost);
  cudaMemcpy(scales_out, scales.data(), h * (w / bs) * 2, cudaMemcpyDeviceToHost);
  if (stats) cudaMemcpy(stats, error.data(), 12, cudaMemcpyDeviceToHost);
  return cudaGetLastError() != cudaSuccess;
}

// device-resident variant: quantizes a device fp16 matrix into device outputs (used to fill the
// reference model's int8 tensors in place)
int ref_quantize_device(void* q_dev, void* scales_dev, const void* in_dev, uint64_t h, uint64_t w, int bs) {
  quantize_absmax_uint8<<<dim3(w / bs, h), std::min(bs, 1024)>>>((uint8_t*)q_dev, (half*)scales_dev, (const half*)in_dev, h,
                                                                w, bs);
  return cudaDeviceSynchronize() != cudaSuccess;
}

int ref_dequantize_absmax_uint8(uint16_t* out, const uint16_t* scales_in, const uint8_t* q_in, uint64_t h, uint64_t w, int bs) {
  tensor4d<half> scales(1, 1, h, w / bs), deq(1, 1, h, w);
  tensor4d<uint8_t> q(1, 1, h, w);
  cudaMemcpy(q.data(), q_in, h * w, cudaMemcpyHostToDevice);
  cudaMemcpy(scales.data(), scales_in, h * (w / bs) * 2, cudaMemcpyHostToDevice);
  dequantize_absmax_uint8<<<dim3(w / bs, h), std::min(bs, 1024)>>>(deq.data(), scales.data(), q.data(), h, w, bs);
  if (cudaDeviceSynchronize() != cudaSuccess) return 1;
  cudaMemcpy(out, deq.data(), h * w * 2, cudaMemcpyDeviceToHost);
  return cudaGetLastError() != cudaSuccess;
}

// the reference's `transform quantize <in> <out> <bs>` on model directories under ./models/
int ref_transform_quantize(const char* in_model, const char* out_model, int bs) {
  mapped_buffer pb(std::string("models/") + in_model + "/params");
  llama_params p;
  if (!pb.is_ok() || !p.load(pb)) return 2;
  return do_quantize(in_model, out_model, p, bs) ? 0 : 1;
}

}  // extern "C"
