// FP32 attention kernels on the CUDA cores.
//
//  * attention_rows_kernel: the reference's example layout q[rows,depth], kt[depth,keys],
//    v[keys,cols]. One warp per query row, keys staged 256 at a time exactly like the
//    staged recurrence the reference emits: each lane owns up to eight scores, warp max,
//    ex2.approx weights kept in shared memory, warp sum, then a probability*value pass in
//    which each lane owns value columns. More than 256 keys chain the stages with the
//    online rescaling of the recurrence.
//  * gqa_f32_kernel: grouped-query attention over [B,H,S,D] tensors with f16 or f32
//    storage, a tiled flash-style kernel (64 queries x 64 keys per step) that keeps every
//    product and the softmax statistics in FP32.
#include <math.h>

#include "dtn_common.cuh"

namespace dtn {

constexpr float kLog2e = 1.4426950408889634f;

// ---------------------------------------------------------------------------------------
// Example-layout attention: one warp per row
// ---------------------------------------------------------------------------------------
constexpr int kRowWarps = 4;
constexpr int kStageKeys = 256;  // 8 rounds of 32 lanes
constexpr int kMaxColGroups = 8; // value columns per lane (cols <= 256)

__global__ void __launch_bounds__(kRowWarps * 32)
attention_rows_kernel(const float* __restrict__ q, const float* __restrict__ kt, const float* __restrict__ v,
                      float* __restrict__ out, int rows, int keys, int depth, int cols, float scale) {
  __shared__ float weights[kRowWarps][kStageKeys];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row = blockIdx.x * kRowWarps + warp;
  if (row >= rows) return;
  const float* qr = q + (int64_t)row * depth;
  float acc[kMaxColGroups];
#pragma unroll
  for (int c = 0; c < kMaxColGroups; ++c) acc[c] = 0.f;
  float run_max = -INFINITY, mass = 0.f;

  for (int k0 = 0; k0 < keys; k0 += kStageKeys) {
    const int stage_keys = min(kStageKeys, keys - k0);
    // scores: lane owns keys k0 + lane + 32*r
    float s[8];
#pragma unroll
    for (int r = 0; r < 8; ++r) s[r] = 0.f;
    for (int d = 0; d < depth; ++d) {
      const float qv = __ldg(qr + d);
      const float* kr = kt + (int64_t)d * keys + k0 + lane;
#pragma unroll
      for (int r = 0; r < 8; ++r)
        if (lane + 32 * r < stage_keys) s[r] = fmaf(qv, __ldg(kr + 32 * r), s[r]);
    }
    float local_max = -INFINITY;
#pragma unroll
    for (int r = 0; r < 8; ++r) {
      s[r] = (lane + 32 * r < stage_keys) ? s[r] * scale : -INFINITY;
      local_max = fmaxf(local_max, s[r]);
    }
    const float stage_max = warp_max(local_max);
    const float new_max = fmaxf(run_max, stage_max);
    const float alpha = (run_max == -INFINITY) ? 0.f : ex2_approx((run_max - new_max) * kLog2e);
    float local_mass = 0.f;
#pragma unroll
    for (int r = 0; r < 8; ++r) {
      if (lane + 32 * r < stage_keys) {
        const float w = ex2_approx((s[r] - new_max) * kLog2e);
        weights[warp][lane + 32 * r] = w;
        local_mass += w;
      }
    }
    mass = mass * alpha + warp_sum(local_mass);
    run_max = new_max;
    __syncwarp();
    // probability * value: lane owns columns lane + 32*c
#pragma unroll
    for (int c = 0; c < kMaxColGroups; ++c) acc[c] *= alpha;
    for (int k = 0; k < stage_keys; ++k) {
      const float w = weights[warp][k];
      const float* vr = v + (int64_t)(k0 + k) * cols + lane;
#pragma unroll
      for (int c = 0; c < kMaxColGroups; ++c)
        if (lane + 32 * c < cols) acc[c] = fmaf(w, __ldg(vr + 32 * c), acc[c]);
    }
    __syncwarp();
  }
  const float inv = rcp_approx(mass);
#pragma unroll
  for (int c = 0; c < kMaxColGroups; ++c)
    if (lane + 32 * c < cols) out[(int64_t)row * cols + lane + 32 * c] = acc[c] * inv;
}

// Same computation with the key and value stages held in shared memory: the CTA's threads fetch a
// stage of SK keys (kt[:, k0:k0+SK] and v[k0:k0+SK, :]) together, then each warp runs the staged
// recurrence of its row out of shared memory. Small problems (the reference's example shapes) are
// latency-bound, and this turns a chain of dependent global loads per row into one round trip per stage.
__device__ __forceinline__ void copy_async_16(float* shared_dst, const float* global_src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((unsigned)__cvta_generic_to_shared(shared_dst)), "l"(global_src)
               : "memory");
}

template <int SK, int CG /*value-column groups of 32 per lane*/>
__global__ void __launch_bounds__(kRowWarps * 32)
attention_staged_kernel(const float* __restrict__ q, const float* __restrict__ kt, const float* __restrict__ v,
                        float* __restrict__ out, int rows, int keys, int depth, int cols, float scale) {
  extern __shared__ __align__(16) float asm_[];
  float* kts = asm_;                         // [depth][SK]
  float* vs = kts + (size_t)depth * SK;      // [SK][cols]
  float* qs = vs + (size_t)SK * cols;        // [kRowWarps][depth]
  float* ws = qs + kRowWarps * depth;        // [kRowWarps][SK]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, tid = threadIdx.x;
  const int row = blockIdx.x * kRowWarps + warp;
  const bool active = row < rows;
  // the CTA's query rows, as asynchronous copies that land with the first stage (a load and a store would hold every
  // thread for one trip to L2 before it could request the stage)
  for (int i = tid; i < kRowWarps * depth; i += kRowWarps * 32) {
    const int r = blockIdx.x * kRowWarps + i / depth;
    const bool in = r < rows;
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"((unsigned)__cvta_generic_to_shared(qs + i)),
                 "l"(in ? q + (int64_t)r * depth + i % depth : q), "r"(in ? 4 : 0)
                 : "memory");
  }
  float acc[CG];
#pragma unroll
  for (int c = 0; c < CG; ++c) acc[c] = 0.f;
  float run_max = -INFINITY, mass = 0.f;
  constexpr int kRounds = SK / 32;
  // vector loads need 16-byte aligned rows of kt and stages of v
  const bool vec_ok = ((reinterpret_cast<uintptr_t>(kt) | reinterpret_cast<uintptr_t>(v)) & 15) == 0 && keys % 4 == 0 &&
                      (SK * cols) % 4 == 0 && (depth * SK) % 4 == 0;

  for (int k0 = 0; k0 < keys; k0 += SK) {
    const int stage_keys = min(SK, keys - k0);
    __syncthreads();   // the previous stage is no longer read (and qs is written before the first use)
    const float* v_stage = v + (int64_t)k0 * cols;
    const int v_count = stage_keys * cols;
    if (vec_ok && stage_keys == SK) {
      // 16-byte asynchronous copies straight into shared memory: every copy of the stage is in flight at once, so the
      // stage costs one trip to L2 however many copies a thread issues (register-staged loads cost one trip per
      // unrolled batch, four for the 128-key example)
      constexpr int kPerRow = SK / 4;
      for (int i = tid; i < depth * kPerRow; i += kRowWarps * 32) {
        const int d = i / kPerRow, k4 = i % kPerRow;
        copy_async_16(kts + d * SK + 4 * k4, kt + (int64_t)d * keys + k0 + 4 * k4);
      }
      for (int i = tid; i < v_count / 4; i += kRowWarps * 32) copy_async_16(vs + 4 * i, v_stage + 4 * i);
    } else {
#pragma unroll 8
      for (int i = tid; i < depth * SK; i += kRowWarps * 32) {
        const int d = i / SK, k = i % SK;
        kts[i] = k < stage_keys ? __ldg(kt + (int64_t)d * keys + k0 + k) : 0.f;
      }
#pragma unroll 8
      for (int i = tid; i < v_count; i += kRowWarps * 32) vs[i] = __ldg(v_stage + i);
    }
    asm volatile("cp.async.commit_group;\n\tcp.async.wait_group 0;" ::: "memory");
    __syncthreads();
    if (active) {
      float s[kRounds];
#pragma unroll
      for (int r = 0; r < kRounds; ++r) s[r] = 0.f;
      const float* qrow = qs + warp * depth;
      int d = 0;
      if (depth % 4 == 0 && kRounds >= 4) {   // four query values per broadcast load; the products are added in the same order
#pragma unroll 2
        for (; d < depth; d += 4) {
          const float4 q4 = *reinterpret_cast<const float4*>(qrow + d);
          const float* kr = kts + d * SK + lane;
#pragma unroll
          for (int r = 0; r < kRounds; ++r) {
            s[r] = fmaf(q4.x, kr[32 * r], s[r]);
            s[r] = fmaf(q4.y, kr[SK + 32 * r], s[r]);
            s[r] = fmaf(q4.z, kr[2 * SK + 32 * r], s[r]);
            s[r] = fmaf(q4.w, kr[3 * SK + 32 * r], s[r]);
          }
        }
      }
      for (; d < depth; ++d) {
        const float qv = qrow[d];
        const float* kr = kts + d * SK + lane;
#pragma unroll
        for (int r = 0; r < kRounds; ++r) s[r] = fmaf(qv, kr[32 * r], s[r]);
      }
      float local_max = -INFINITY;
#pragma unroll
      for (int r = 0; r < kRounds; ++r) {
        s[r] = (lane + 32 * r < stage_keys) ? s[r] * scale : -INFINITY;
        local_max = fmaxf(local_max, s[r]);
      }
      const float new_max = fmaxf(run_max, warp_max(local_max));
      const float alpha = (run_max == -INFINITY) ? 0.f : ex2_approx((run_max - new_max) * kLog2e);
      float local_mass = 0.f;
#pragma unroll
      for (int r = 0; r < kRounds; ++r) {
        const float w = (lane + 32 * r < stage_keys) ? ex2_approx((s[r] - new_max) * kLog2e) : 0.f;
        ws[warp * SK + lane + 32 * r] = w;
        local_mass += w;
      }
      mass = mass * alpha + warp_sum(local_mass);
      run_max = new_max;
      __syncwarp();
#pragma unroll
      for (int c = 0; c < CG; ++c) acc[c] *= alpha;
      const float* wrow = ws + warp * SK;
      int k = 0;
      if (CG == 1 && stage_keys == SK) {   // one column group: four weights per broadcast load, the same order of additions (slower with two groups)
#pragma unroll 4
        for (; k < SK; k += 4) {
          const float4 w4 = *reinterpret_cast<const float4*>(wrow + k);
          const float* vr = vs + k * cols + lane;
#pragma unroll
          for (int c = 0; c < CG; ++c)
            if (lane + 32 * c < cols) {
              acc[c] = fmaf(w4.x, vr[32 * c], acc[c]);
              acc[c] = fmaf(w4.y, vr[cols + 32 * c], acc[c]);
              acc[c] = fmaf(w4.z, vr[2 * cols + 32 * c], acc[c]);
              acc[c] = fmaf(w4.w, vr[3 * cols + 32 * c], acc[c]);
            }
        }
      }
      for (; k < stage_keys; ++k) {
        const float w = wrow[k];
        const float* vr = vs + k * cols + lane;
#pragma unroll
        for (int c = 0; c < CG; ++c)
          if (lane + 32 * c < cols) acc[c] = fmaf(w, vr[32 * c], acc[c]);
      }
    }
  }
  if (active) {
    const float inv = rcp_approx(mass);
#pragma unroll
    for (int c = 0; c < CG; ++c)
      if (lane + 32 * c < cols) out[(int64_t)row * cols + lane + 32 * c] = acc[c] * inv;
  }
}

static size_t staged_smem_bytes(int sk, int64_t depth, int64_t cols) {
  return sizeof(float) * ((size_t)depth * sk + (size_t)sk * cols + (size_t)kRowWarps * depth + (size_t)kRowWarps * sk);
}

template <int SK, int CG>
static int attention_staged_launch_cg(const float* q, const float* kt, const float* v, float* out, int64_t rows, int64_t keys,
                                   int64_t depth, int64_t cols, float scale, cudaStream_t s) {
  const size_t smem = staged_smem_bytes(SK, depth, cols);
  auto kernel = attention_staged_kernel<SK, CG>;
  static thread_local int attr_dev = -1;
  static thread_local size_t attr_bytes = 0;
  int dev = 0;
  DTN_CUDA_CHECK(cudaGetDevice(&dev));
  if (smem > 48 * 1024 && (attr_dev != dev || attr_bytes < smem)) {
    DTN_CUDA_CHECK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    attr_dev = dev;
    attr_bytes = 200 * 1024;
  }
  const int64_t blocks = (rows + kRowWarps - 1) / kRowWarps;
  kernel<<<(unsigned)blocks, kRowWarps * 32, smem, s>>>(q, kt, v, out, (int)rows, (int)keys, (int)depth, (int)cols, scale);
  DTN_LAUNCH_CHECK("attention_staged_kernel");
  return DTN_OK;
}

template <int SK>
static int attention_staged_launch(const float* q, const float* kt, const float* v, float* out, int64_t rows, int64_t keys,
                                   int64_t depth, int64_t cols, float scale, cudaStream_t s) {
  if (cols <= 32) return attention_staged_launch_cg<SK, 1>(q, kt, v, out, rows, keys, depth, cols, scale, s);
  if (cols <= 64) return attention_staged_launch_cg<SK, 2>(q, kt, v, out, rows, keys, depth, cols, scale, s);
  if (cols <= 96) return attention_staged_launch_cg<SK, 3>(q, kt, v, out, rows, keys, depth, cols, scale, s);
  if (cols <= 128) return attention_staged_launch_cg<SK, 4>(q, kt, v, out, rows, keys, depth, cols, scale, s);
  if (cols <= 192) return attention_staged_launch_cg<SK, 6>(q, kt, v, out, rows, keys, depth, cols, scale, s);
  return attention_staged_launch_cg<SK, 8>(q, kt, v, out, rows, keys, depth, cols, scale, s);
}

// ---------------------------------------------------------------------------------------
// Grouped-query attention, FP32 math, tiled
// ---------------------------------------------------------------------------------------
constexpr int G_BM = 64, G_BN = 64, G_THREADS = 256;

template <typename T>
__device__ __forceinline__ float load_as_f32(const T* p);
template <>
__device__ __forceinline__ float load_as_f32<float>(const float* p) { return __ldg(p); }
template <>
__device__ __forceinline__ float load_as_f32<__half>(const __half* p) {
  return __half2float(__ldg(p));
}

template <typename T, int D>
__global__ void __launch_bounds__(G_THREADS)
gqa_f32_kernel(const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v,
               float* __restrict__ out, int Hq, int Hkv, int S, float scale, int group_begin) {
  extern __shared__ __align__(16) float gsm[];
  float* Qt = gsm;                         // [D][G_BM]
  float* Kt = Qt + D * G_BM;               // [D][G_BN + 4]
  float* Vs = Kt + D * (G_BN + 4);         // [G_BN][D]
  float* Ps = Vs + G_BN * D;               // [G_BM][G_BN + 4]
  constexpr int KT_LD = G_BN + 4, PS_LD = G_BN + 4;

  const int heads_per_group = Hq / Hkv;
  const int group = group_begin + blockIdx.y / heads_per_group;  // (batch, kv head)
  const int b = group / Hkv, hkv = group % Hkv;
  const int hq = hkv * heads_per_group + blockIdx.y % heads_per_group;
  const int q0 = blockIdx.x * G_BM;
  const T* qh = q + ((int64_t)(b * Hq + hq) * S) * D;
  const T* kh = k + ((int64_t)(b * Hkv + hkv) * S) * D;
  const T* vh = v + ((int64_t)(b * Hkv + hkv) * S) * D;
  float* oh = out + ((int64_t)(b * Hq + hq) * S) * D;

  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;

  // Q tile, transposed, pre-multiplied by nothing (scale is applied to the score as the
  // reference does).
  for (int i = tid; i < G_BM * D; i += G_THREADS) {
    const int r = i / D, d = i % D;
    Qt[d * G_BM + r] = (q0 + r < S) ? load_as_f32(qh + (int64_t)(q0 + r) * D + d) : 0.f;
  }

  constexpr int OC = D / 16;  // output columns per thread: tx*4.. in blocks of 64
  float o[4][OC];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < OC; ++j) o[i][j] = 0.f;
  float row_max[4], row_mass[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) { row_max[i] = -INFINITY; row_mass[i] = 0.f; }

  for (int n0 = 0; n0 < S; n0 += G_BN) {
    __syncthreads();
    for (int i = tid; i < G_BN * D; i += G_THREADS) {
      const int r = i / D, d = i % D;
      const bool in = n0 + r < S;
      Kt[d * KT_LD + r] = in ? load_as_f32(kh + (int64_t)(n0 + r) * D + d) : 0.f;
      Vs[r * D + d] = in ? load_as_f32(vh + (int64_t)(n0 + r) * D + d) : 0.f;
    }
    __syncthreads();
    // scores: 4 rows (ty*4+i) x 4 keys (tx*4+j)
    float s[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) s[i][j] = 0.f;
#pragma unroll 8
    for (int d = 0; d < D; ++d) {
      const float4 a = *reinterpret_cast<const float4*>(Qt + d * G_BM + ty * 4);
      const float4 bb = *reinterpret_cast<const float4*>(Kt + d * KT_LD + tx * 4);
      const float av[4] = {a.x, a.y, a.z, a.w}, bv[4] = {bb.x, bb.y, bb.z, bb.w};
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) s[i][j] = fmaf(av[i], bv[j], s[i][j]);
    }
    float alpha[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float m = -INFINITY;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        s[i][j] = (n0 + tx * 4 + j < S) ? s[i][j] * scale : -INFINITY;
        m = fmaxf(m, s[i][j]);
      }
      // the 16 threads sharing ty hold one row: butterfly over tx (low four lane bits)
#pragma unroll
      for (int off = 8; off > 0; off >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, off));
      const float new_max = fmaxf(row_max[i], m);
      alpha[i] = (row_max[i] == -INFINITY) ? 0.f : ex2_approx((row_max[i] - new_max) * kLog2e);
      float sum = 0.f;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float w = ex2_approx((s[i][j] - new_max) * kLog2e);
        s[i][j] = w;
        sum += w;
      }
#pragma unroll
      for (int off = 8; off > 0; off >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, off);
      row_mass[i] = row_mass[i] * alpha[i] + sum;
      row_max[i] = new_max;
      *reinterpret_cast<float4*>(Ps + (ty * 4 + i) * PS_LD + tx * 4) = make_float4(s[i][0], s[i][1], s[i][2], s[i][3]);
    }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < OC; ++j) o[i][j] *= alpha[i];
#pragma unroll 4
    for (int n = 0; n < G_BN; ++n) {
      float p[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) p[i] = Ps[(ty * 4 + i) * PS_LD + n];
#pragma unroll
      for (int jb = 0; jb < OC / 4; ++jb) {
        const float4 vv = *reinterpret_cast<const float4*>(Vs + n * D + jb * 64 + tx * 4);
        const float vj[4] = {vv.x, vv.y, vv.z, vv.w};
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
          for (int j = 0; j < 4; ++j) o[i][jb * 4 + j] = fmaf(p[i], vj[j], o[i][jb * 4 + j]);
      }
    }
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int r = q0 + ty * 4 + i;
    if (r >= S) continue;
    const float inv = rcp_approx(row_mass[i]);
#pragma unroll
    for (int jb = 0; jb < OC / 4; ++jb)
      *reinterpret_cast<float4*>(oh + (int64_t)r * D + jb * 64 + tx * 4) =
          make_float4(o[i][jb * 4 + 0] * inv, o[i][jb * 4 + 1] * inv, o[i][jb * 4 + 2] * inv, o[i][jb * 4 + 3] * inv);
  }
}

template <typename T, int D>
static int gqa_f32_launch_d(const void* q, const void* k, const void* v, float* out, int64_t Hq, int64_t Hkv,
                            int64_t S, float scale, int64_t gb, int64_t ge, cudaStream_t s) {
  constexpr size_t smem = sizeof(float) * (D * G_BM + D * (G_BN + 4) + G_BN * D + G_BM * (G_BN + 4));
  auto kernel = gqa_f32_kernel<T, D>;
  static thread_local int attr_dev = -1;
  int dev = 0;
  DTN_CUDA_CHECK(cudaGetDevice(&dev));
  if (attr_dev != dev) {
    DTN_CUDA_CHECK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    attr_dev = dev;
  }
  const int64_t heads = (ge - gb) * (Hq / Hkv);
  DTN_REQUIRE(heads <= 65535, DTN_ERR_UNSUPPORTED, "gqa: too many heads for one launch");
  dim3 grid((unsigned)((S + G_BM - 1) / G_BM), (unsigned)heads);
  kernel<<<grid, G_THREADS, smem, s>>>(static_cast<const T*>(q), static_cast<const T*>(k),
                                       static_cast<const T*>(v), out, (int)Hq, (int)Hkv, (int)S, scale, (int)gb);
  DTN_LAUNCH_CHECK("gqa_f32_kernel");
  return DTN_OK;
}

int gqa_f32_launch(const void* q, const void* k, const void* v, float* out, int64_t Hq, int64_t Hkv, int64_t S,
                   int64_t D, float scale, int storage, int64_t gb, int64_t ge, cudaStream_t s) {
#define DTN_GQA_CASE(DD)                                                                              \
  case DD:                                                                                            \
    return storage == DTN_STORAGE_F16                                                                 \
               ? gqa_f32_launch_d<__half, DD>(q, k, v, out, Hq, Hkv, S, scale, gb, ge, s)               \
               : gqa_f32_launch_d<float, DD>(q, k, v, out, Hq, Hkv, S, scale, gb, ge, s);
  switch (D) {
    DTN_GQA_CASE(64)
    DTN_GQA_CASE(128)
    default:
      set_error("gqa: head_dim %lld is not supported by the FP32 kernel (64 or 128)", (long long)D);
      return DTN_ERR_UNSUPPORTED;
  }
#undef DTN_GQA_CASE
}

}  // namespace dtn

extern "C" int dtn_attention_f32(const float* q, const float* kt, const float* v, float* out, int64_t rows,
                                 int64_t keys, int64_t depth, int64_t cols, float scale, void* stream) {
  using namespace dtn;
  DTN_REQUIRE(rows >= 0 && keys >= 0 && depth >= 0 && cols >= 0, DTN_ERR_INVALID, "attention: negative extent");
  if (rows == 0 || cols == 0) return DTN_OK;
  DTN_REQUIRE(q && kt && v && out, DTN_ERR_INVALID, "attention: null pointer");
  DTN_REQUIRE(keys > 0, DTN_ERR_INVALID, "attention: at least one key is required");
  DTN_REQUIRE(cols <= 32 * kMaxColGroups, DTN_ERR_UNSUPPORTED, "attention: at most %d value columns",
              32 * kMaxColGroups);
  DTN_REQUIRE(rows < (1LL << 31) && keys < (1LL << 31) && depth < (1LL << 31), DTN_ERR_UNSUPPORTED,
              "attention: extents must fit 31 bits");
  // Stage keys through shared memory when a stage fits (the largest stage of 256, 128, 64 or 32 keys
  // within 200 KiB); otherwise stream from global memory.
  constexpr size_t kStageLimit = 200 * 1024;
  const int64_t wanted = keys < 32 ? 32 : keys;
  if (wanted > 128 && staged_smem_bytes(256, depth, cols) <= kStageLimit)
    return attention_staged_launch<256>(q, kt, v, out, rows, keys, depth, cols, scale, as_stream(stream));
  if (wanted > 64 && staged_smem_bytes(128, depth, cols) <= kStageLimit)
    return attention_staged_launch<128>(q, kt, v, out, rows, keys, depth, cols, scale, as_stream(stream));
  if (wanted > 32 && staged_smem_bytes(64, depth, cols) <= kStageLimit)
    return attention_staged_launch<64>(q, kt, v, out, rows, keys, depth, cols, scale, as_stream(stream));
  if (staged_smem_bytes(32, depth, cols) <= kStageLimit)
    return attention_staged_launch<32>(q, kt, v, out, rows, keys, depth, cols, scale, as_stream(stream));
  const int64_t blocks = (rows + kRowWarps - 1) / kRowWarps;
  attention_rows_kernel<<<(unsigned)blocks, kRowWarps * 32, 0, as_stream(stream)>>>(
      q, kt, v, out, (int)rows, (int)keys, (int)depth, (int)cols, scale);
  DTN_LAUNCH_CHECK("attention_rows_kernel");
  return DTN_OK;
}
