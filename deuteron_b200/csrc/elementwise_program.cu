// Fused elementwise expressions over f16 / f32 buffers: one pass over memory for a whole chain of
// operators (for example the reference's f16 "affine" kernel, f16(x * scale + bias), and its
// "cancellation" kernel, f16((x + y) - x), both computed in explicit FP32).
//
// The expression arrives as a short register program (at most 24 instructions over 8 virtual
// registers). Every thread interprets it on 8 consecutive elements at a time: the operand
// decode is uniform across the grid (no divergence) and is paid once per 8 elements, so the
// kernel stays bandwidth-bound. Vector inputs are read with 128-bit loads, one-element inputs
// are broadcast, arithmetic is FP32 with one rounding per operator (no contraction into fma, so
// results equal the reference's operator-by-operator NumPy expectation), and the result is
// narrowed to f16 with round-to-nearest-even when the output buffer is f16.
#include "dtn_common.cuh"
#include "program.cuh"

namespace dtn {

constexpr int kProgMaxInstr = 24;
constexpr int kProgRegs = 8;
constexpr int kProgMaxInputs = 6;

struct EwProgram {
  int n_inputs;                      // registers 0..n_inputs-1 are loaded from the inputs
  int n_instr;
  int out_reg;
  int out_f16;                       // 1: narrow the result to f16
  const void* input[kProgMaxInputs];
  unsigned char input_f16[kProgMaxInputs];
  unsigned char input_scalar[kProgMaxInputs];   // 1: one-element buffer, broadcast
  unsigned char op[kProgMaxInstr], dst[kProgMaxInstr], a[kProgMaxInstr], b[kProgMaxInstr];
};

// W = 8: vector body (every vector pointer 16-byte aligned at `first`); W = 1: scalar elements.
template <int W>
__global__ void __launch_bounds__(256)
ew_program_kernel(const EwProgram prog, void* __restrict__ out, int64_t first, int64_t count) {
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t item = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; item < count; item += stride) {
    const int64_t base = first + item * W;
    RegFile<kProgRegs, W> regs;
#pragma unroll
    for (int i = 0; i < kProgMaxInputs; ++i) {
      if (i >= prog.n_inputs) break;
      float v[W];
      if (prog.input_scalar[i]) {
        const float s = prog.input_f16[i] ? __half2float(*static_cast<const __half*>(prog.input[i]))
                                          : *static_cast<const float*>(prog.input[i]);
#pragma unroll
        for (int e = 0; e < W; ++e) v[e] = s;
      } else if (prog.input_f16[i]) {
        const __half* p = static_cast<const __half*>(prog.input[i]) + base;
        if constexpr (W == 8) {
          uint4 raw = ld_stream_u4(reinterpret_cast<const uint4*>(p));
          const __half2* h = reinterpret_cast<const __half2*>(&raw);
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float2 f = __half22float2(h[e]);
            v[2 * e] = f.x;
            v[2 * e + 1] = f.y;
          }
        } else {
          v[0] = __half2float(p[0]);
        }
      } else {
        const float* p = static_cast<const float*>(prog.input[i]) + base;
        if constexpr (W == 8) {
          const float4 lo = ld_stream_f4(reinterpret_cast<const float4*>(p));
          const float4 hi = ld_stream_f4(reinterpret_cast<const float4*>(p) + 1);
          v[0] = lo.x; v[1] = lo.y; v[2] = lo.z; v[3] = lo.w;
          v[4] = hi.x; v[5] = hi.y; v[6] = hi.z; v[7] = hi.w;
        } else {
          v[0] = p[0];
        }
      }
      regs.put(i, v);
    }
    for (int n = 0; n < prog.n_instr; ++n) {
      float a[W], b[W], d[W];
      regs.get(prog.a[n], a);
      regs.get(prog.b[n], b);
      const int op = prog.op[n];
#pragma unroll
      for (int e = 0; e < W; ++e) d[e] = prog_apply(op, a[e], b[e]);
      regs.put(prog.dst[n], d);
    }
    float result[W];
    regs.get(prog.out_reg, result);
    if (prog.out_f16) {
      __half* q = static_cast<__half*>(out) + base;
      if constexpr (W == 8) {
        uint4 packed;
        __half2* h = reinterpret_cast<__half2*>(&packed);
#pragma unroll
        for (int e = 0; e < 4; ++e) h[e] = __floats2half2_rn(result[2 * e], result[2 * e + 1]);
        st_stream_u4(reinterpret_cast<uint4*>(q), packed);
      } else {
        q[0] = __float2half_rn(result[0]);
      }
    } else {
      float* q = static_cast<float*>(out) + base;
      if constexpr (W == 8) {
        st_stream_f4(reinterpret_cast<float4*>(q), make_float4(result[0], result[1], result[2], result[3]));
        st_stream_f4(reinterpret_cast<float4*>(q) + 1, make_float4(result[4], result[5], result[6], result[7]));
      } else {
        q[0] = result[0];
      }
    }
  }
}

// ---------------------------------------------------------------------------------------
// Chain form: every instruction combines the previous result with an input (or with itself), as in
// x * scale + bias, relu(x) * y or (x + y) - x. The inputs are loaded up front (all loads in flight
// together), the operator of a step is decoded once per 8 elements outside the lane loop, and no
// register file is indexed at run time. Programs of any other shape use the interpreter above.
// ---------------------------------------------------------------------------------------
constexpr int kEwChainMax = 8;
struct EwChain {
  int n, start;                 // start: the input the running value begins as
  unsigned long long steps;     // one byte per step: operator (bits 0-3), operand input (bits 4-6, 7 = the running value), swap (bit 7)
};

template <int W>
__device__ __forceinline__ void ew_load_input(const EwProgram& prog, int i, int64_t base, float (&v)[W]) {
  if (prog.input_scalar[i]) {
    const float s = prog.input_f16[i] ? __half2float(*static_cast<const __half*>(prog.input[i]))
                                      : __ldg(static_cast<const float*>(prog.input[i]));
#pragma unroll
    for (int e = 0; e < W; ++e) v[e] = s;
  } else if (prog.input_f16[i]) {
    const __half* p = static_cast<const __half*>(prog.input[i]) + base;
    if constexpr (W == 8) {
      uint4 raw = ld_stream_u4(reinterpret_cast<const uint4*>(p));
      const __half2* h = reinterpret_cast<const __half2*>(&raw);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 f = __half22float2(h[e]);
        v[2 * e] = f.x;
        v[2 * e + 1] = f.y;
      }
    } else {
      v[0] = __half2float(p[0]);
    }
  } else {
    const float* p = static_cast<const float*>(prog.input[i]) + base;
    if constexpr (W == 8) {
      const float4 lo = ld_stream_f4(reinterpret_cast<const float4*>(p));
      const float4 hi = ld_stream_f4(reinterpret_cast<const float4*>(p) + 1);
      v[0] = lo.x; v[1] = lo.y; v[2] = lo.z; v[3] = lo.w;
      v[4] = hi.x; v[5] = hi.y; v[6] = hi.z; v[7] = hi.w;
    } else {
      v[0] = p[0];
    }
  }
}

template <int OP, int W>
__device__ __forceinline__ void ew_chain_step(float (&acc)[W], const float (&o)[W], bool swap) {
#pragma unroll
  for (int e = 0; e < W; ++e) {
    if constexpr (OP == DTN_EW_SUB) acc[e] = swap ? __fsub_rn(o[e], acc[e]) : __fsub_rn(acc[e], o[e]);
    else if constexpr (OP == DTN_EW_DIV) acc[e] = swap ? __fdividef(o[e], acc[e]) : __fdividef(acc[e], o[e]);
    else acc[e] = prog_apply(OP, acc[e], o[e]);
  }
}

// One step with the operand held in registers: the operator switch is a uniform branch.
template <int W>
__device__ __forceinline__ void ew_chain_apply(int op, float (&acc)[W], const float (&o)[W], bool swap) {
#define DTN_EW_CASE(OP) case OP: ew_chain_step<OP, W>(acc, o, swap); break;
  switch (op) {
    DTN_EW_CASE(DTN_EW_ADD) DTN_EW_CASE(DTN_EW_SUB) DTN_EW_CASE(DTN_EW_MUL) DTN_EW_CASE(DTN_EW_DIV) DTN_EW_CASE(DTN_EW_MAX)
    DTN_EW_CASE(DTN_EW_MIN) DTN_EW_CASE(DTN_EW_RELU) DTN_EW_CASE(DTN_EW_EXP) DTN_EW_CASE(DTN_EW_SQRT) DTN_EW_CASE(DTN_EW_RSQRT)
    DTN_EW_CASE(DTN_EW_RCP) DTN_EW_CASE(DTN_EW_NEG) DTN_EW_CASE(DTN_EW_ABS)
    default: break;   // copy
  }
#undef DTN_EW_CASE
}

// NIN: an upper bound of the number of inputs (1, 2, 3 or 6), so that a program with one or two inputs does not hold
// registers for six and more items are in flight per SM.
template <int W, int NIN>
__global__ void __launch_bounds__(256)
ew_chain_kernel(const EwProgram prog, const EwChain chain, void* __restrict__ out, int64_t first, int64_t count) {
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  // one-element inputs are the same for every item: read them once
  float constant[NIN];
#pragma unroll
  for (int i = 0; i < NIN; ++i) {
    constant[i] = 0.0f;
    if (i < prog.n_inputs && prog.input_scalar[i])
      constant[i] = prog.input_f16[i] ? __half2float(*static_cast<const __half*>(prog.input[i])) : __ldg(static_cast<const float*>(prog.input[i]));
  }
  for (int64_t item = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; item < count; item += stride) {
    const int64_t base = first + item * W;
    float in[NIN][W];
#pragma unroll
    for (int i = 0; i < NIN; ++i) {
      if (i < prog.n_inputs) {
        if (prog.input_scalar[i]) {
#pragma unroll
          for (int e = 0; e < W; ++e) in[i][e] = constant[i];
        } else {
          ew_load_input<W>(prog, i, base, in[i]);
        }
      }
    }
    float acc[W];
    switch (chain.start) {
#define DTN_EW_START(I) case I: _Pragma("unroll") for (int e = 0; e < W; ++e) acc[e] = in[I < NIN ? I : 0][e]; break;
      DTN_EW_START(1) DTN_EW_START(2) DTN_EW_START(3) DTN_EW_START(4) DTN_EW_START(5)
      default: DTN_EW_START(0)
#undef DTN_EW_START
    }
    unsigned long long steps = chain.steps;
    for (int s = 0; s < chain.n; ++s, steps >>= 8) {
      const int op = (int)(steps & 15), operand = (int)((steps >> 4) & 7);
      const bool swap = ((steps >> 7) & 1) != 0;
      switch (operand) {
        case 0: if constexpr (0 < NIN) ew_chain_apply<W>(op, acc, in[0], swap); break;
        case 1: if constexpr (1 < NIN) ew_chain_apply<W>(op, acc, in[1], swap); break;
        case 2: if constexpr (2 < NIN) ew_chain_apply<W>(op, acc, in[2], swap); break;
        case 3: if constexpr (3 < NIN) ew_chain_apply<W>(op, acc, in[3], swap); break;
        case 4: if constexpr (4 < NIN) ew_chain_apply<W>(op, acc, in[4], swap); break;
        case 5: if constexpr (5 < NIN) ew_chain_apply<W>(op, acc, in[5], swap); break;
        default: {
          float self[W];
#pragma unroll
          for (int e = 0; e < W; ++e) self[e] = acc[e];
          ew_chain_apply<W>(op, acc, self, swap);
        }
      }
    }
    if (prog.out_f16) {
      __half* q = static_cast<__half*>(out) + base;
      if constexpr (W == 8) {
        uint4 packed;
        __half2* h = reinterpret_cast<__half2*>(&packed);
#pragma unroll
        for (int e = 0; e < 4; ++e) h[e] = __floats2half2_rn(acc[2 * e], acc[2 * e + 1]);
        st_stream_u4(reinterpret_cast<uint4*>(q), packed);
      } else {
        q[0] = __float2half_rn(acc[0]);
      }
    } else {
      float* q = static_cast<float*>(out) + base;
      if constexpr (W == 8) {
        st_stream_f4(reinterpret_cast<float4*>(q), make_float4(acc[0], acc[1], acc[2], acc[3]));
        st_stream_f4(reinterpret_cast<float4*>(q) + 1, make_float4(acc[4], acc[5], acc[6], acc[7]));
      } else {
        q[0] = acc[0];
      }
    }
  }
}

// Chain form of `prog`, if it has one: the first instruction reads inputs only, every later one reads the previous
// result and an input no instruction has overwritten (or the previous result twice).
static bool ew_chain_of(const EwProgram& prog, EwChain* chain) {
  chain->n = 0;
  chain->start = 0;
  chain->steps = 0;
  if (prog.n_instr == 0) {
    chain->start = prog.out_reg;
    return prog.out_reg < prog.n_inputs;
  }
  if (prog.n_instr > kEwChainMax) return false;
  bool written[kProgRegs] = {false};
  int running = -1;
  for (int n = 0; n < prog.n_instr; ++n) {
    const int op = prog.op[n], a = prog.a[n], b = prog.b[n];
    const bool binary = op <= DTN_EW_MIN;
    auto is_input = [&](int r) { return r < prog.n_inputs && !written[r]; };
    int other = 7;   // the running value
    bool swap = false;
    if (n == 0) {
      if (!is_input(a) || (binary && !is_input(b))) return false;
      chain->start = a;
      if (binary) other = b;
    } else if (!binary) {
      if (a != running) return false;
    } else if (a == running) {
      other = b;
    } else if (b == running) {
      other = a;
      swap = true;
    } else {
      return false;
    }
    if (binary && n > 0) {
      if (other == running) other = 7;
      else if (!is_input(other)) return false;
    }
    chain->steps |= (unsigned long long)((op & 15) | ((other & 7) << 4) | (swap ? 128 : 0)) << (8 * chain->n);
    ++chain->n;
    running = prog.dst[n];
    written[running] = true;
  }
  return prog.out_reg == running;
}

}  // namespace dtn

extern "C" int dtn_elementwise_program(const unsigned char* ops, const unsigned char* dsts, const unsigned char* as,
                                       const unsigned char* bs, int n_instr, const void* const* inputs,
                                       const unsigned char* input_f16, const unsigned char* input_scalar, int n_inputs,
                                       int out_reg, void* out, int out_f16, int64_t n, void* stream) {
  using namespace dtn;
  DTN_REQUIRE(n >= 0, DTN_ERR_INVALID, "elementwise program: negative n");
  DTN_REQUIRE(n_instr >= 0 && n_instr <= kProgMaxInstr, DTN_ERR_UNSUPPORTED, "elementwise program: at most %d instructions",
              kProgMaxInstr);
  DTN_REQUIRE(n_inputs >= 1 && n_inputs <= kProgMaxInputs, DTN_ERR_UNSUPPORTED, "elementwise program: 1..%d inputs",
              kProgMaxInputs);
  DTN_REQUIRE(out_reg >= 0 && out_reg < kProgRegs, DTN_ERR_INVALID, "elementwise program: bad output register");
  if (n == 0) return DTN_OK;
  DTN_REQUIRE(out && inputs && input_f16 && input_scalar && (n_instr == 0 || (ops && dsts && as && bs)), DTN_ERR_INVALID,
              "elementwise program: null pointer");
  EwProgram prog = {};
  prog.n_inputs = n_inputs;
  prog.n_instr = n_instr;
  prog.out_reg = out_reg;
  prog.out_f16 = out_f16 ? 1 : 0;
  const void* vec_ptrs[kProgMaxInputs + 1];
  int vec_sizes[kProgMaxInputs + 1];
  int vec_count = 0;
  for (int i = 0; i < n_inputs; ++i) {
    DTN_REQUIRE(inputs[i] != nullptr, DTN_ERR_INVALID, "elementwise program: input %d is null", i);
    const int size = input_f16[i] ? 2 : 4;
    DTN_REQUIRE(aligned_to(inputs[i], size), DTN_ERR_INVALID, "elementwise program: input %d is misaligned", i);
    prog.input[i] = inputs[i];
    prog.input_f16[i] = input_f16[i] ? 1 : 0;
    prog.input_scalar[i] = input_scalar[i] ? 1 : 0;
    if (!input_scalar[i]) {
      vec_ptrs[vec_count] = inputs[i];
      vec_sizes[vec_count++] = size;
    }
  }
  for (int k = 0; k < n_instr; ++k) {
    DTN_REQUIRE(ops[k] <= DTN_EW_COPY && dsts[k] < kProgRegs && as[k] < kProgRegs && bs[k] < kProgRegs, DTN_ERR_INVALID,
                "elementwise program: instruction %d is malformed", k);
    prog.op[k] = ops[k];
    prog.dst[k] = dsts[k];
    prog.a[k] = as[k];
    prog.b[k] = bs[k];
  }
  const int out_size = out_f16 ? 2 : 4;
  DTN_REQUIRE(aligned_to(out, out_size), DTN_ERR_INVALID, "elementwise program: output is misaligned");
  vec_ptrs[vec_count] = out;
  vec_sizes[vec_count++] = out_size;
  cudaStream_t s = as_stream(stream);
  // smallest head (in elements) after which every vector pointer is 16-byte aligned
  int head = -1;
  for (int h = 0; h < 16 && head < 0; ++h) {
    bool ok = true;
    for (int i = 0; i < vec_count && ok; ++i)
      ok = ((reinterpret_cast<uintptr_t>(vec_ptrs[i]) + (uintptr_t)h * vec_sizes[i]) & 15) == 0;
    if (ok) head = h;
  }
  auto grid_for = [](int64_t items) {
    int64_t blocks = (items + 255) / 256;
    const int64_t cap = (int64_t)sm_count() * 32;
    return (unsigned)(blocks < 1 ? 1 : (blocks > cap ? cap : blocks));
  };
  EwChain chain;
  const bool chained = ew_chain_of(prog, &chain);
  auto scalar_launch = [&](unsigned grid, unsigned block, int64_t first, int64_t count) {
    if (chained)
      ew_chain_kernel<1, kProgMaxInputs><<<grid, block, 0, s>>>(prog, chain, out, first, count);
    else
      ew_program_kernel<1><<<grid, block, 0, s>>>(prog, out, first, count);
  };
  if (head < 0 || n < 64) {
    scalar_launch(grid_for(n), 256, 0, n);
    DTN_LAUNCH_CHECK("elementwise program (scalar)");
    return DTN_OK;
  }
  const int64_t body = (n - head) / 8;
  const int64_t tail_start = head + body * 8;
  if (head > 0) {
    scalar_launch(1, 32, 0, head);
    DTN_LAUNCH_CHECK("elementwise program (head)");
  }
  if (body > 0) {
    // small problems: 64-thread blocks spread the work over more SMs
    const unsigned block = body < 4096 ? 64 : 256;
    const unsigned grid = body < 4096 ? (unsigned)((body + 63) / 64) : grid_for(body);
    if (chained && n_inputs <= 1)
      ew_chain_kernel<8, 1><<<grid, block, 0, s>>>(prog, chain, out, head, body);
    else if (chained && n_inputs <= 2)
      ew_chain_kernel<8, 2><<<grid, block, 0, s>>>(prog, chain, out, head, body);
    else if (chained && n_inputs <= 3)
      ew_chain_kernel<8, 3><<<grid, block, 0, s>>>(prog, chain, out, head, body);
    else if (chained)
      ew_chain_kernel<8, kProgMaxInputs><<<grid, block, 0, s>>>(prog, chain, out, head, body);
    else
      ew_program_kernel<8><<<grid, block, 0, s>>>(prog, out, head, body);
    DTN_LAUNCH_CHECK("elementwise program (body)");
  }
  if (tail_start < n) {
    scalar_launch(1, 32, tail_start, n - tail_start);
    DTN_LAUNCH_CHECK("elementwise program (tail)");
  }
  return DTN_OK;
}
