"""Functor snippets: the C++ a scalar code generator would print for the user's
functions, one per collective operation.

In accelerate-cuda the scalar functions of a program are turned into C by
``Data/Array/Accelerate/CUDA/CodeGen.hs:338-821`` and pasted into a skeleton
template; here each snippet defines a struct that a skeleton header of
``csrc/skeletons/`` is instantiated with.  ``ALL`` lists what ``build.py``
compiles ahead of time: the five benchmark configurations plus the small
programs the tests use, so a fresh machine finds them in the in-tree kernel
cache.

The five configurations are written from their plain-English definitions:
  dot      foldAll (+) 0 (zipWith (*) xs ys)                      Float
  scan_add scanl / scanl' / scanl1 / scanr.. (+) on Int32
  hist     permute (+) zeros (\\i -> index1 (keys!i)) (fill n 1)  Int32
  blur     stencil, 3x3 weights 1/16 [1 2 1; 2 4 2; 1 2 1]        Float
  blackscholes  map over (spot, strike, years) -> (call, put)     Float
  rowsum   fold (+) 0 over the innermost dimension                Float
"""
from __future__ import annotations

from dataclasses import dataclass


@dataclass(frozen=True)
class KernelSpec:
    skeleton: str   # "map", "fold_all", "fold_dim", "fold_seg", "scan", "permute", "permute_smem", "stencil", "stencil2"
    functor: str    # name of the struct defined by `source`
    source: str
    flags: str = ""


_D = "static __device__ __forceinline__"

# --------------------------------------------------------------------- folds
# A recognised (+) on Float accumulates in double and rounds once, which keeps
# every float32 sum within one rounding of the exact value.
DOT = KernelSpec("fold_all", "Dot", f"""
struct Dot : accb::Fold<float, double> {{
    using In = accb::types<float, float>;
    {_D} float get(const accb::Env &, long long, float x, float y) {{ return x * y; }}
    {_D} double lift(float x) {{ return (double)x; }}
    {_D} double combine(double a, double b) {{ return a + b; }}
}};
""")

# the same dot product with a float32 accumulator: what pasting the user's
# (+) :: Float -> Float -> Float verbatim gives
DOT_F32ACC = KernelSpec("fold_all", "DotF", f"""
struct DotF : accb::Fold<float> {{
    using In = accb::types<float, float>;
    {_D} float get(const accb::Env &, long long, float x, float y) {{ return x * y; }}
    {_D} float combine(float a, float b) {{ return a + b; }}
}};
""")

SUM_F32 = KernelSpec("fold_all", "SumF", f"""
struct SumF : accb::Fold<float, double> {{
    using In = accb::types<float>;
    {_D} float get(const accb::Env &, long long, float x) {{ return x; }}
    {_D} double combine(double a, double b) {{ return a + b; }}
}};
""")

SUM_I32 = KernelSpec("fold_all", "SumI", f"""
struct SumI : accb::Fold<int> {{
    using In = accb::types<int>;
    {_D} int get(const accb::Env &, long long, int x) {{ return x; }}
    {_D} int combine(int a, int b) {{ return (int)((unsigned)a + (unsigned)b); }}
}};
""")

MAX_I32 = KernelSpec("fold_all", "MaxI", f"""
struct MaxI : accb::Fold<int> {{
    using In = accb::types<int>;
    {_D} int get(const accb::Env &, long long, int x) {{ return x; }}
    {_D} int combine(int a, int b) {{ return max(a, b); }}
}};
""")

# fold over pairs: (value, index) arg-max, two SoA components in and out
ARGMAX = KernelSpec("fold_all", "ArgMax", f"""
struct VI {{ float v; int i; }};
struct ArgMax {{
    typedef VI elem; typedef VI acc;
    using In = accb::types<float>;
    using Out = accb::types<float, int>;
    {_D} VI get(const accb::Env &, long long i, float x) {{ VI r; r.v = x; r.i = (int)i; return r; }}
    {_D} VI lift(VI x) {{ return x; }}
    {_D} VI lower(VI x) {{ return x; }}
    {_D} VI combine(VI a, VI b) {{ return (b.v > a.v || (b.v == a.v && b.i < a.i)) ? b : a; }}
    {_D} void put(VI r, float &v, int &i) {{ v = r.v; i = r.i; }}
}};
""")

ROWSUM = KernelSpec("fold_dim", "RowSum", f"""
struct RowSum : accb::Fold<float, double> {{
    using In = accb::types<float>;
    {_D} float get(const accb::Env &, long long, float x) {{ return x; }}
    {_D} double combine(double a, double b) {{ return a + b; }}
}};
""")

ROWSUM_I32 = KernelSpec("fold_dim", "RowSumI", f"""
struct RowSumI : accb::Fold<int> {{
    using In = accb::types<int>;
    {_D} int get(const accb::Env &, long long, int x) {{ return x; }}
    {_D} int combine(int a, int b) {{ return (int)((unsigned)a + (unsigned)b); }}
}};
""")

ROWMIN_I32 = KernelSpec("fold_dim", "RowMinI", f"""
struct RowMinI : accb::Fold<int> {{
    using In = accb::types<int>;
    {_D} int get(const accb::Env &, long long, int x) {{ return x; }}
    {_D} int combine(int a, int b) {{ return min(a, b); }}
}};
""")

SEGSUM_I32 = KernelSpec("fold_seg", "SegSumI", f"""
struct SegSumI : accb::Fold<int> {{
    using In = accb::types<int>;
    {_D} int get(const accb::Env &, long long, int x) {{ return x; }}
    {_D} int combine(int a, int b) {{ return (int)((unsigned)a + (unsigned)b); }}
}};
""")

SEGSUM_F32 = KernelSpec("fold_seg", "SegSumF", f"""
struct SegSumF : accb::Fold<float, double> {{
    using In = accb::types<float>;
    {_D} float get(const accb::Env &, long long, float x) {{ return x; }}
    {_D} double combine(double a, double b) {{ return a + b; }}
}};
""")

# sparse matrix x dense vector in CSR form: foldSeg (+) 0 (zipWith (*) vals (gather cols vec)) rowOffsets.
# Environment: (vals, cols) zipped element-wise, then the dense vector as a free array variable.
SMVM = KernelSpec("fold_seg", "Smvm", f"""
struct Smvm : accb::Fold<float, double> {{
    using In = accb::types<float, int>;
    {_D} float get(const accb::Env &env, long long, float v, int c) {{ return v * env.in<float>(2)[c]; }}
    {_D} double combine(double a, double b) {{ return a + b; }}
}};
""")

# row-wise dot products of two matrices: fold (+) 0 (zipWith (*) a b)
ROWDOT = KernelSpec("fold_dim", "RowDot", f"""
struct RowDot : accb::Fold<float, double> {{
    using In = accb::types<float, float>;
    {_D} float get(const accb::Env &, long long, float x, float y) {{ return x * y; }}
    {_D} double combine(double a, double b) {{ return a + b; }}
}};
""")

# --------------------------------------------------------------------- scans
SCAN_ADD_I32 =KernelSpec("scan", "AddI", f"""
struct AddI : accb::Scan<int> {{
    using In = accb::types<int>;
    {_D} int get(const accb::Env &, long long, int x) {{ return x; }}
    {_D} int combine(int a, int b) {{ return (int)((unsigned)a + (unsigned)b); }}
}};
""")

SCAN_ADD_I64 = KernelSpec("scan", "AddL", f"""
struct AddL : accb::Scan<long long> {{
    using In = accb::types<long long>;
    {_D} long long get(const accb::Env &, long long, long long x) {{ return x; }}
    {_D} long long combine(long long a, long long b) {{ return (long long)((unsigned long long)a + (unsigned long long)b); }}
}};
""")

SCAN_ADD_F32 = KernelSpec("scan", "AddF", f"""
struct AddF : accb::Scan<float> {{
    using In = accb::types<float>;
    {_D} float get(const accb::Env &, long long, float x) {{ return x; }}
    {_D} float combine(float a, float b) {{ return a + b; }}
}};
""")

SCAN_MAX_I32 = KernelSpec("scan", "MaxS", f"""
struct MaxS : accb::Scan<int> {{
    using In = accb::types<int>;
    {_D} int get(const accb::Env &, long long, int x) {{ return x; }}
    {_D} int combine(int a, int b) {{ return max(a, b); }}
}};
""")

# Composition of affine maps x -> a*x + b over Word32: associative but NOT
# commutative, and a two-component (SoA) value: exercises value order and the
# record form of the tile status.  combine(f, g) = "f then g".
SCAN_AFFINE = KernelSpec("scan", "Affine", f"""
struct AB {{ unsigned a, b; }};
struct Affine {{
    typedef AB elem; typedef AB acc;
    using In = accb::types<unsigned, unsigned>;
    using Out = accb::types<unsigned, unsigned>;
    {_D} AB get(const accb::Env &, long long, unsigned a, unsigned b) {{ AB r; r.a = a; r.b = b; return r; }}
    {_D} AB combine(AB f, AB g) {{ AB r; r.a = g.a * f.a; r.b = g.a * f.b + g.b; return r; }}
    {_D} void put(AB r, unsigned &a, unsigned &b) {{ a = r.a; b = r.b; }}
}};
""")

# ------------------------------------------------------------------- permute
HIST = KernelSpec("permute_smem", "Hist", f"""
struct Hist : accb::Permute<int, accb::Atomic::Add> {{
    using In = accb::types<int>;
    {_D} long long index(const accb::Env &, long long, int key) {{ return key; }}
    {_D} int get(const accb::Env &, long long, int) {{ return 1; }}
    {_D} int combine(int x, int y) {{ return (int)((unsigned)x + (unsigned)y); }}
    {_D} int identity() {{ return 0; }}
}};
""")

# the same histogram straight into global memory (no privatisation)
HIST_GLOBAL = KernelSpec("permute", "HistG", f"""
struct HistG : accb::Permute<int, accb::Atomic::Add> {{
    using In = accb::types<int>;
    {_D} long long index(const accb::Env &, long long, int key) {{ return key; }}
    {_D} int get(const accb::Env &, long long, int) {{ return 1; }}
    {_D} int combine(int x, int y) {{ return (int)((unsigned)x + (unsigned)y); }}
}};
""")

# weighted histogram: keys and a manifest weights array
HIST_WEIGHTED = KernelSpec("permute_smem", "HistW", f"""
struct HistW : accb::Permute<int, accb::Atomic::Add> {{
    using In = accb::types<int, int>;
    {_D} long long index(const accb::Env &, long long, int key, int) {{ return key; }}
    {_D} int get(const accb::Env &, long long, int, int w) {{ return w; }}
    {_D} int combine(int x, int y) {{ return (int)((unsigned)x + (unsigned)y); }}
    {_D} int identity() {{ return 0; }}
}};
""")

# float max through a compare-and-swap loop
SCATTER_MAX_F32 = KernelSpec("permute", "MaxF", f"""
struct MaxF : accb::Permute<float, accb::Atomic::Cas> {{
    using In = accb::types<int, float>;
    {_D} long long index(const accb::Env &, long long, int key, float) {{ return key; }}
    {_D} float get(const accb::Env &, long long, int, float v) {{ return v; }}
    {_D} float combine(float x, float y) {{ return fmaxf(x, y); }}
}};
""")

# a true permutation: the combiner ignores the old value, so no atomics at all
SCATTER = KernelSpec("permute", "Scatter", f"""
struct Scatter : accb::Permute<int, accb::Atomic::None> {{
    using In = accb::types<int, int>;
    {_D} long long index(const accb::Env &, long long, int dst, int) {{ return dst; }}
    {_D} int get(const accb::Env &, long long, int, int v) {{ return v; }}
    {_D} int combine(int x, int) {{ return x; }}
}};
""")

# pairs (sum, count) per key: a tuple value, updated under the per-element lock
SCATTER_PAIR = KernelSpec("permute", "SumCount", f"""
struct SC {{ int s, c; }};
struct SumCount {{
    typedef SC elem;
    static constexpr accb::Atomic atomic = accb::Atomic::Lock;
    using In = accb::types<int, int>;
    using Out = accb::types<int, int>;
    {_D} long long index(const accb::Env &, long long, int key, int) {{ return key; }}
    {_D} SC get(const accb::Env &, long long, int, int v) {{ SC r; r.s = v; r.c = 1; return r; }}
    {_D} SC combine(SC x, SC y) {{ SC r; r.s = x.s + y.s; r.c = x.c + y.c; return r; }}
    {_D} void put(SC r, int &s, int &c) {{ s = r.s; c = r.c; }}
    {_D} SC take(const int &s, const int &c) {{ SC r; r.s = s; r.c = c; return r; }}
}};
""")

# ------------------------------------------------------------------ stencils
BLUR = KernelSpec("stencil", "Blur", f"""
struct Blur : accb::Stencil<float, float, 1, 1> {{
    {_D} float apply(const accb::Env &, const float (&t)[3][3]) {{
        return 0.0625f * t[0][0] + 0.125f * t[0][1] + 0.0625f * t[0][2]
             + 0.125f  * t[1][0] + 0.25f  * t[1][1] + 0.125f  * t[1][2]
             + 0.0625f * t[2][0] + 0.125f * t[2][1] + 0.0625f * t[2][2];
    }}
}};
""")

LAPLACE = KernelSpec("stencil", "Laplace", f"""
struct Laplace : accb::Stencil<float, float, 1, 1> {{
    {_D} float apply(const accb::Env &, const float (&t)[3][3]) {{
        return t[0][1] + t[1][0] + t[1][2] + t[2][1] - 4.0f * t[1][1];
    }}
}};
""")

# 5x5 box filter: radius 2 in both directions
BOX5 = KernelSpec("stencil", "Box5", f"""
struct Box5 : accb::Stencil<float, float, 2, 2> {{
    {_D} float apply(const accb::Env &, const float (&t)[5][5]) {{
        float s = 0.0f;
        for (int y = 0; y < 5; ++y) for (int x = 0; x < 5; ++x) s += t[y][x];
        return s * 0.04f;
    }}
}};
""")

# rank-1, 3 taps
SMOOTH1D = KernelSpec("stencil", "Smooth1", f"""
struct Smooth1 : accb::Stencil<float, float, 0, 1> {{
    {_D} float apply(const accb::Env &, const float (&t)[1][3]) {{
        return 0.25f * t[0][0] + 0.5f * t[0][1] + 0.25f * t[0][2];
    }}
}};
""")

# rank 3: a 3x3x3 neighbourhood with 27 different weights (w[dz][dy][dx] = (9 dz + 3 dy + dx + 1) / 378), so that
# a tap read from the wrong plane, row or column changes the result
WEIGHTED27 = KernelSpec("stencil3", "Weighted27", f"""
struct Weighted27 : accb::Stencil3<float, float, 1, 1, 1> {{
    {_D} float apply(const accb::Env &, const float (&t)[3][3][3]) {{
        float s = 0.0f;
        for (int z = 0; z < 3; ++z) for (int y = 0; y < 3; ++y) for (int x = 0; x < 3; ++x)
            s += (float)(9 * z + 3 * y + x + 1) * t[z][y][x];
        return s * (1.0f / 378.0f);
    }}
}};
""")

# rank 3: the 7-point Laplacian
LAPLACE3 = KernelSpec("stencil3", "Laplace3", f"""
struct Laplace3 : accb::Stencil3<float, float, 1, 1, 1> {{
    static constexpr bool uses(int z, int y, int x) {{ return (z == 1) + (y == 1) + (x == 1) >= 2; }}  // centre + 6 axis neighbours
    {_D} float apply(const accb::Env &, const float (&t)[3][3][3]) {{
        return t[0][1][1] + t[2][1][1] + t[1][0][1] + t[1][2][1] + t[1][1][0] + t[1][1][2] - 6.0f * t[1][1][1];
    }}
}};
""")

STENCIL2_SUM = KernelSpec("stencil2", "Cross2", f"""
struct Cross2 : accb::Stencil<float, float, 1, 1> {{
    {_D} float apply(const accb::Env &, const float (&a)[3][3], const float (&b)[3][3]) {{
        return a[1][1] + 0.5f * (a[1][0] + a[1][2]) + 0.25f * (b[0][1] + b[2][1]) - b[1][1];
    }}
}};
""")

# ---------------------------------------------------------------------- maps
# European call and put.  erf is not an Accelerate primitive
# (CodeGen.hs:406-476): it enters as a foreign scalar function
# (CodeGen.hs:793-805), here the CUDA math library's erff.  The kernel is
# compiled with -use_fast_math (approximate division, log, exp and square
# root), which turns this functor from ALU-bound into memory-bound; measured
# against the float64 oracle the prices then need an absolute floor of 3e-6
# beside the 1e-5 relative tolerance.
BLACKSCHOLES = KernelSpec("map", "BlackScholes", f"""
struct BlackScholes {{
    using In = accb::types<float, float, float>;
    using Out = accb::types<float, float>;
    {_D} float cnd(float d) {{ return 0.5f + 0.5f * erff(0.70710678f * d); }}
    {_D} void apply(const accb::Env &, long long, float s, float k, float t, float &call, float &put) {{
        const float r = 0.02f, v = 0.30f;
        const float sq = sqrtf(t), vsq = v * sq;
        const float d1 = (logf(s / k) + (r + 0.5f * v * v) * t) / vsq;
        const float d2 = d1 - vsq;
        const float kexp = k * expf(-r * t);
        const float n1 = cnd(d1), n2 = cnd(d2);
        call = s * n1 - kexp * n2;
        put = kexp * (1.0f - n2) - s * (1.0f - n1);
    }}
}};
""", flags="-use_fast_math")

# the same functor with the accurate math library (IEEE division, logf, expf,
# sqrtf, erfcf): ALU-bound on B200, kept for comparison
BLACKSCHOLES_ACCURATE = KernelSpec("map", "BlackScholesA", f"""
struct BlackScholesA {{
    using In = accb::types<float, float, float>;
    using Out = accb::types<float, float>;
    {_D} float cnd(float d) {{ return 0.5f * erfcf(-0.70710678f * d); }}
    {_D} void apply(const accb::Env &, long long, float s, float k, float t, float &call, float &put) {{
        const float r = 0.02f, v = 0.30f;
        const float sq = sqrtf(t), vsq = v * sq;
        const float d1 = (logf(s / k) + (r + 0.5f * v * v) * t) / vsq;
        const float d2 = d1 - vsq;
        const float kexp = k * expf(-r * t);
        const float n1 = cnd(d1), n2 = cnd(d2);
        call = s * n1 - kexp * n2;
        put = kexp * (1.0f - n2) - s * (1.0f - n1);
    }}
}};
""")

# zipWith with user scalars: out = a*x + y, a read from the scalar block
# one value in, one out, and the element's index: out[i] = 2 x + (i mod 5)
SCALE_PLUS_INDEX = KernelSpec("map", "ScalePlusIndex", f"""
struct ScalePlusIndex {{
    using In = accb::types<float>;
    using Out = accb::types<float>;
    {_D} void apply(const accb::Env &, long long i, float x, float &o) {{ o = 2.0f * x + (float)(i % 5); }}
}};
""")

SAXPY = KernelSpec("map", "Saxpy", f"""
struct Saxpy {{
    using In = accb::types<float, float>;
    using Out = accb::types<float>;
    {_D} void apply(const accb::Env &env, long long, float x, float y, float &o) {{
        o = env.scalar<float>(0) * x + y;
    }}
}};
""")

# zipWith (+) on Int32: merges the partial destinations of a permute (+) that ran on several GPUs
ZIP_ADD_I32 = KernelSpec("map", "ZipAddI", f"""
struct ZipAddI {{
    using In = accb::types<int, int>;
    using Out = accb::types<int>;
    {_D} void apply(const accb::Env &, long long, int x, int y, int &o) {{ o = (int)((unsigned)x + (unsigned)y); }}
}};
""")

# generate: a function of the index only
IOTA_SQ = KernelSpec("map", "IotaSq", f"""
struct IotaSq {{
    using In = accb::types<>;
    using Out = accb::types<int>;
    {_D} void apply(const accb::Env &, long long i, int &o) {{ o = (int)(i * i + 1); }}
}};
""")

# backpermute / transform: gather through an index array (environment slot 0 =
# indices, read element-wise; slot 1 = the source, gathered)
GATHER = KernelSpec("map", "Gather", f"""
struct Gather {{
    using In = accb::types<int>;
    using Out = accb::types<int>;
    {_D} void apply(const accb::Env &env, long long, int j, int &o) {{ o = env.in<int>(1)[j]; }}
}};
""")

# transpose of a rank-2 array by index arithmetic (backpermute swap)
TRANSPOSE = KernelSpec("map", "Transpose", f"""
struct Transpose {{
    using In = accb::types<>;
    using Out = accb::types<float>;
    {_D} void apply(const accb::Env &env, long long i, float &o) {{
        int y, x;
        accb::from_index2(env.out_dim(0), i, y, x);
        o = env.in<float>(0)[accb::to_index2(env.dim(0, 0), x, y)];
    }}
}};
""")

# element types of every width, to exercise the 4 / 8 / 16 / 32-byte vector paths
WIDEN = KernelSpec("map", "Widen", f"""
struct Widen {{
    using In = accb::types<signed char, short, double>;
    using Out = accb::types<long long, unsigned char>;
    {_D} void apply(const accb::Env &, long long, signed char a, short b, double c, long long &o, unsigned char &f) {{
        o = (long long)a * b + (long long)c;
        f = (unsigned char)(a > 0);
    }}
}};
""")

ALL = {name: spec for name, spec in globals().items() if isinstance(spec, KernelSpec)}
