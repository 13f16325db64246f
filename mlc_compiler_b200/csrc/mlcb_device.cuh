// Device library prepended to every generated translation unit (sm_100a).
//
// The generated kernels are specialisations: shapes, strides, grids and vector
// widths are literals in their text.  What they share lives here -- packed
// global-memory access (up to 128 bits per instruction), exact narrow-float
// rounding, NaN-propagating min/max, and the cross-lane reductions (sub-warp and
// warp butterflies over shuffles, one shared-memory hop for a CTA-wide row).
//
// Arithmetic conventions (they are what parity with the torch reference backend
// rests on): fp16/bf16 operands are widened to fp32 on load and all float math
// is fp32 with IEEE division and square root and no fused multiply-add
// contraction (the module is compiled with --fmad=false, never with fast-math);
// a value whose IR dtype is fp16/bf16 is held in a float register that always
// contains an exactly representable narrow value.  Kernels that store only
// fp16/bf16 may use the SFU-based forms further down (error ~1e-6 relative,
// invisible after the narrow rounding); kernels with an fp32 output never do.
#pragma once

#include <cuda_fp16.h>
#include <cuda_bf16.h>

typedef long long i64;
typedef unsigned long long u64;

#define MLCB_INF_F   __int_as_float(0x7f800000)
#define MLCB_NINF_F  __int_as_float(0xff800000)
#define MLCB_NAN_F   __int_as_float(0x7fc00000)
#define MLCB_INF_D   __longlong_as_double(0x7ff0000000000000LL)
#define MLCB_NINF_D  __longlong_as_double(0xfff0000000000000LL)
#define MLCB_NAN_D   __longlong_as_double(0x7ff8000000000000LL)

// Programmatic dependent launch: a kernel launched with the stream-serialisation
// attribute may start while its predecessor drains.  Before the wait it may only
// read memory that no kernel of the schedule writes (weights, biases, masks: the
// emitter places exactly those loads there) and must store nothing.  Without
// the attribute both are no-ops.
#if defined(MLCB_PDL) && MLCB_PDL
#define MLCB_GRID_WAIT()    asm volatile("griddepcontrol.wait;" ::: "memory")
#define MLCB_GRID_TRIGGER() asm volatile("griddepcontrol.launch_dependents;" ::: "memory")
#else
#define MLCB_GRID_WAIT()
#define MLCB_GRID_TRIGGER()
#endif

// ---------------------------------------------------------------------------
// narrow-float rounding and element conversion
// ---------------------------------------------------------------------------
__device__ __forceinline__ float mlcb_rn_f16(float x) { return __half2float(__float2half_rn(x)); }
__device__ __forceinline__ float mlcb_rn_bf16(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }

template <typename T> struct mlcb_elem;  // storage type -> register type
template <> struct mlcb_elem<__half> {
    typedef float reg;
    static __device__ __forceinline__ float get(__half v) { return __half2float(v); }
    static __device__ __forceinline__ __half put(float v) { return __float2half_rn(v); }
};
template <> struct mlcb_elem<__nv_bfloat16> {
    typedef float reg;
    static __device__ __forceinline__ float get(__nv_bfloat16 v) { return __bfloat162float(v); }
    static __device__ __forceinline__ __nv_bfloat16 put(float v) { return __float2bfloat16_rn(v); }
};
#define MLCB_PLAIN_ELEM(T)                                                        \
    template <> struct mlcb_elem<T> {                                             \
        typedef T reg;                                                            \
        static __device__ __forceinline__ T get(T v) { return v; }                \
        static __device__ __forceinline__ T put(T v) { return v; }                \
    };
MLCB_PLAIN_ELEM(float)
MLCB_PLAIN_ELEM(double)
MLCB_PLAIN_ELEM(i64)
MLCB_PLAIN_ELEM(int)
MLCB_PLAIN_ELEM(short)
MLCB_PLAIN_ELEM(signed char)
MLCB_PLAIN_ELEM(unsigned char)
MLCB_PLAIN_ELEM(bool)

// ---------------------------------------------------------------------------
// packed global access: W consecutive elements, W * sizeof(T) bytes, aligned to
// min(32, W * sizeof(T)).  The emitter proves the alignment from the index map
// before it asks for a width.
// ---------------------------------------------------------------------------
template <int BYTES> struct mlcb_word;
template <> struct mlcb_word<1>  { typedef unsigned char  type; };
template <> struct mlcb_word<2>  { typedef unsigned short type; };
template <> struct mlcb_word<4>  { typedef unsigned int   type; };
template <> struct mlcb_word<8>  { typedef uint2          type; };
template <> struct mlcb_word<16> { typedef uint4          type; };
// 256-bit global accesses are new with sm_100 (ld/st.global.v4.b64): one
// instruction moves 32 bytes per lane, 1 KB per warp.
struct alignas(32) mlcb_u256 { unsigned long long x[4]; };
template <> struct mlcb_word<32> { typedef mlcb_u256      type; };

template <typename W> __device__ __forceinline__ W mlcb_ld_word(const W* p) { return *p; }
template <typename W> __device__ __forceinline__ void mlcb_st_word(W* p, const W& v) { *p = v; }
template <> __device__ __forceinline__ mlcb_u256 mlcb_ld_word<mlcb_u256>(const mlcb_u256* p) {
    mlcb_u256 v;
    asm volatile("ld.global.v4.u64 {%0, %1, %2, %3}, [%4];"
                 : "=l"(v.x[0]), "=l"(v.x[1]), "=l"(v.x[2]), "=l"(v.x[3]) : "l"(p));
    return v;
}
template <> __device__ __forceinline__ void mlcb_st_word<mlcb_u256>(mlcb_u256* p, const mlcb_u256& v) {
    asm volatile("st.global.v4.u64 [%4], {%0, %1, %2, %3};"
                 :: "l"(v.x[0]), "l"(v.x[1]), "l"(v.x[2]), "l"(v.x[3]), "l"(p) : "memory");
}

template <typename T, int W>
struct mlcb_pack {
    static constexpr int BYTES = W * (int)sizeof(T);
    // bytes per instruction: 32 when the pack is a whole number of 256-bit words
    static constexpr int CHUNK = (BYTES % 32 == 0) ? 32 : (BYTES > 16 ? 16 : BYTES);
    static constexpr int N = BYTES / CHUNK;
    typedef typename mlcb_word<CHUNK>::type word;
    union { word w[N]; T e[W]; };
    __device__ __forceinline__ mlcb_pack() {}
};

template <typename T, int W>
__device__ __forceinline__ void mlcb_load(const T* __restrict__ p,
                                          typename mlcb_elem<T>::reg (&dst)[W]) {
    mlcb_pack<T, W> u;
    typedef typename mlcb_pack<T, W>::word word;
    const word* q = reinterpret_cast<const word*>(p);
#pragma unroll
    for (int i = 0; i < mlcb_pack<T, W>::N; ++i) u.w[i] = mlcb_ld_word(q + i);
#pragma unroll
    for (int i = 0; i < W; ++i) dst[i] = mlcb_elem<T>::get(u.e[i]);
}

// The same access in two halves: the packed words now (they can sit in a
// quarter of the registers while other work proceeds -- e.g. weights fetched
// before the grid-dependency wait), the widening to register type at the use.
template <typename T, int W>
__device__ __forceinline__ void mlcb_load_raw(const T* __restrict__ p, mlcb_pack<T, W>& u) {
    typedef typename mlcb_pack<T, W>::word word;
    const word* q = reinterpret_cast<const word*>(p);
#pragma unroll
    for (int i = 0; i < mlcb_pack<T, W>::N; ++i) u.w[i] = mlcb_ld_word(q + i);
}
template <typename T, int W>
__device__ __forceinline__ void mlcb_unpack(const mlcb_pack<T, W>& u,
                                            typename mlcb_elem<T>::reg (&dst)[W]) {
#pragma unroll
    for (int i = 0; i < W; ++i) dst[i] = mlcb_elem<T>::get(u.e[i]);
}

// Same, into elements [at, at + W) of a wider register array.
template <typename T, int W, int V>
__device__ __forceinline__ void mlcb_load_at(const T* __restrict__ p,
                                             typename mlcb_elem<T>::reg (&dst)[V], int at) {
    typename mlcb_elem<T>::reg tmp[W];
    mlcb_load<T, W>(p, tmp);
#pragma unroll
    for (int i = 0; i < W; ++i) dst[at + i] = tmp[i];
}

// Register array -> packed storage words.  fp16/bf16 convert two registers per
// instruction (cvt.rn.f16x2.f32 / cvt.rn.bf16x2.f32).
template <typename T, int W>
struct mlcb_packer {
    static __device__ __forceinline__ void run(mlcb_pack<T, W>& u,
                                               const typename mlcb_elem<T>::reg (&src)[W]) {
#pragma unroll
        for (int i = 0; i < W; ++i) u.e[i] = mlcb_elem<T>::put(src[i]);
    }
};
template <int W>
struct mlcb_packer<__half, W> {
    static __device__ __forceinline__ void run(mlcb_pack<__half, W>& u, const float (&src)[W]) {
        if constexpr (W % 2 == 0) {
            __half2* h = reinterpret_cast<__half2*>(u.e);
#pragma unroll
            for (int i = 0; i < W / 2; ++i) h[i] = __floats2half2_rn(src[2 * i], src[2 * i + 1]);
        } else {
#pragma unroll
            for (int i = 0; i < W; ++i) u.e[i] = __float2half_rn(src[i]);
        }
    }
};
template <int W>
struct mlcb_packer<__nv_bfloat16, W> {
    static __device__ __forceinline__ void run(mlcb_pack<__nv_bfloat16, W>& u, const float (&src)[W]) {
        if constexpr (W % 2 == 0) {
            __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(u.e);
#pragma unroll
            for (int i = 0; i < W / 2; ++i) h[i] = __floats2bfloat162_rn(src[2 * i], src[2 * i + 1]);
        } else {
#pragma unroll
            for (int i = 0; i < W; ++i) u.e[i] = __float2bfloat16_rn(src[i]);
        }
    }
};

template <typename T, int W>
__device__ __forceinline__ void mlcb_store(T* __restrict__ p,
                                           const typename mlcb_elem<T>::reg (&src)[W]) {
    mlcb_pack<T, W> u;
    typedef typename mlcb_pack<T, W>::word word;
    mlcb_packer<T, W>::run(u, src);
    word* q = reinterpret_cast<word*>(p);
#pragma unroll
    for (int i = 0; i < mlcb_pack<T, W>::N; ++i) mlcb_st_word(q + i, u.w[i]);
}

template <typename T, int W, int V>
__device__ __forceinline__ void mlcb_store_at(T* __restrict__ p,
                                              const typename mlcb_elem<T>::reg (&src)[V], int at) {
    typename mlcb_elem<T>::reg tmp[W];
#pragma unroll
    for (int i = 0; i < W; ++i) tmp[i] = src[at + i];
    mlcb_store<T, W>(p, tmp);
}

// Row id of a gathered operand, forced into the table: an id outside [0, n)
// reads a wrong row instead of memory that is not the table's.
__device__ __forceinline__ long long mlcb_clamp_index(long long v, long long n) {
    return v < 0 ? 0 : (v >= n ? n - 1 : v);
}

template <typename T>
__device__ __forceinline__ typename mlcb_elem<T>::reg mlcb_load1(const T* __restrict__ p) {
    return mlcb_elem<T>::get(*p);
}
template <typename T>
__device__ __forceinline__ void mlcb_store1(T* __restrict__ p, typename mlcb_elem<T>::reg v) {
    *p = mlcb_elem<T>::put(v);
}

// ---------------------------------------------------------------------------
// scalar functions whose CUDA spelling is not a plain operator
// ---------------------------------------------------------------------------
// torch.maximum / torch.minimum / amax / amin propagate NaN; fmaxf does not.
template <typename T> __device__ __forceinline__ T mlcb_max(T a, T b) { return (a > b || a != a) ? a : b; }
template <typename T> __device__ __forceinline__ T mlcb_min(T a, T b) { return (a < b || a != a) ? a : b; }
__device__ __forceinline__ float  mlcb_sigmoid(float x)  { return 1.0f / (1.0f + expf(-x)); }
__device__ __forceinline__ double mlcb_sigmoid(double x) { return 1.0 / (1.0 + exp(-x)); }
__device__ __forceinline__ float  mlcb_rsqrt(float x)  { return 1.0f / sqrtf(x); }
__device__ __forceinline__ double mlcb_rsqrt(double x) { return 1.0 / sqrt(x); }
// SFU-based forms used only where the result is rounded to fp16/bf16 before it
// is stored (absolute error about 2e-7, far below half-precision resolution).
// The .ftz variants are single MUFU instructions; the non-ftz intrinsics wrap
// them in subnormal scaling that costs more than the operation itself.
__device__ __forceinline__ float mlcb_ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ float mlcb_rcp_fast(float x) {
    float y;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ float mlcb_lg2(float x) {
    float y;
    asm("lg2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ float mlcb_rcp(float x) { return __frcp_rn(x); }
__device__ __forceinline__ float mlcb_exp_fast(float x) { return mlcb_ex2(x * 1.4426950408889634f); }
__device__ __forceinline__ float mlcb_log_fast(float x) { return mlcb_lg2(x) * 0.6931471805599453f; }
__device__ __forceinline__ float mlcb_div_fast(float a, float b) { return a * mlcb_rcp_fast(b); }
__device__ __forceinline__ float mlcb_tanh_fast(float x) {
    // 1 - 2 / (1 + e^(2x)): exact limits at +-inf, NaN propagates
    return fmaf(-2.0f, mlcb_rcp_fast(1.0f + mlcb_ex2(x * 2.8853900817779268f)), 1.0f);
}
__device__ __forceinline__ float mlcb_sigmoid_fast(float x) {
    return mlcb_rcp_fast(1.0f + mlcb_ex2(x * -1.4426950408889634f));
}
__device__ __forceinline__ float mlcb_erf_fast(float x) {
    // Abramowitz & Stegun 7.1.26, |error| <= 1.5e-7
    const float ax = fabsf(x);
    const float t = mlcb_rcp_fast(fmaf(0.3275911f, ax, 1.0f));
    float p = fmaf(1.061405429f, t, -1.453152027f);
    p = fmaf(p, t, 1.421413741f);
    p = fmaf(p, t, -0.284496736f);
    p = fmaf(p, t, 0.254829592f);
    const float r = fmaf(-(p * t), mlcb_ex2(ax * ax * -1.4426950408889634f), 1.0f);
    return copysignf(r, x);
}
__device__ __forceinline__ i64 mlcb_ipow(i64 b, i64 e) {
    if (e < 0) return (b == 1) ? 1 : ((b == -1) ? ((e & 1) ? -1 : 1) : 0);
    i64 r = 1;
    while (e) { if (e & 1) r *= b; b *= b; e >>= 1; }
    return r;
}
template <typename T> __device__ __forceinline__ T mlcb_iabs(T x) {
    if constexpr (T(-1) > T(0)) return x;        // unsigned
    else return x < 0 ? -x : x;
}

// ---------------------------------------------------------------------------
// reductions
// ---------------------------------------------------------------------------
struct mlcb_op_sum  { template <typename T> static __device__ __forceinline__ T f(T a, T b) { return a + b; } };
struct mlcb_op_prod { template <typename T> static __device__ __forceinline__ T f(T a, T b) { return a * b; } };
struct mlcb_op_max  { template <typename T> static __device__ __forceinline__ T f(T a, T b) { return mlcb_max(a, b); } };
struct mlcb_op_min  { template <typename T> static __device__ __forceinline__ T f(T a, T b) { return mlcb_min(a, b); } };

template <typename T> __device__ __forceinline__ T mlcb_shfl_xor(T v, int m) { return __shfl_xor_sync(0xffffffffu, v, m); }
template <> __device__ __forceinline__ bool mlcb_shfl_xor<bool>(bool v, int m) { return __shfl_xor_sync(0xffffffffu, (int)v, m) != 0; }

// Butterfly over G consecutive lanes (G a power of two, 1..32).  Every lane of
// the group ends with the group's result, so a row statistic needs no broadcast.
template <typename OP, int G, typename T>
__device__ __forceinline__ T mlcb_group_reduce(T v) {
#pragma unroll
    for (int m = G >> 1; m > 0; m >>= 1) v = OP::f(v, mlcb_shfl_xor(v, m));
    return v;
}

// A row owned by a whole CTA of NW warps: butterfly inside each warp, one hop
// through shared memory, every thread combines the NW partials in the same
// order (deterministic, and all threads hold the result).  `slot` points at NW
// elements that no other reduction of the kernel reuses before the next barrier.
template <typename OP, int NW, typename T>
__device__ __forceinline__ T mlcb_cta_reduce(T v, T* slot) {
    v = mlcb_group_reduce<OP, 32>(v);
    if ((threadIdx.x & 31) == 0) slot[threadIdx.x >> 5] = v;
    __syncthreads();
    T r = slot[0];
#pragma unroll
    for (int w = 1; w < NW; ++w) r = OP::f(r, slot[w]);
    return r;
}
