/*
 * CPU oracle for the TOSA reference model's CONV2D / DEPTHWISE_CONV2D / MATMUL /
 * RESCALE / CLAMP / ADD / MAX_POOL2D / AVG_POOL2D evaluation.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is a plain-C restatement of the reference
 * interpreter's arithmetic, used to check the CUDA library and to time a CPU
 * baseline.  Nothing in the shipped library links, loads or calls it.
 *
 * Pinning: the restatement is checked against the reference's own known-answer
 * tests (reference_model/test/ref_model_tests/tensor_ops_tests.cpp:622-683,
 * :736-822; type_conversion_tests.cpp:322-405) and against the two convolution
 * example graphs shipped with the reference (examples/test_conv2d_1x1_1x32x32x8_*),
 * whose expected outputs are committed as fixtures.
 *
 * Storage follows the reference's host containers (src/ops/template_types.h:67-147):
 * every integer tensor is int32_t per element, fp16/bf16/fp32 tensors are float,
 * precise-mode tensors are double.  All arrays are row-major in TOSA shape order
 * (NHWC activations, OHWI conv weights, [KH,KW,C,M] depthwise weights).
 *
 * Each function names the reference lines it follows.  `nthreads > 1` only splits
 * the outermost output loops with OpenMP; per-element arithmetic and accumulation
 * order are unchanged.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

/* graph status values, include/graph_status.h:18-23 */
#define ORC_VALID 0
#define ORC_UNPREDICTABLE 1
#define ORC_ERROR 2

#define ORC_API __attribute__((visibility("default")))

/* ------------------------------------------------------------------------- */
/* fp16 / bf16 rounding (what fpTrunc<Dtype> does, src/arith_util.h:206-230).  */
/* Round-to-nearest-even; the reference delegates to ct::cfloat casts.         */
/* ------------------------------------------------------------------------- */
static float orc_round_bf16(float f)
{
    uint32_t u;
    memcpy(&u, &f, 4);
    if ((u & 0x7f800000u) == 0x7f800000u)
    {
        if (u & 0x007fffffu)
            u |= 0x00400000u; /* keep NaN a NaN after truncation */
        u &= 0xffff0000u;
    }
    else
    {
        uint32_t lsb = (u >> 16) & 1u;
        u += 0x7fffu + lsb;
        u &= 0xffff0000u;
    }
    memcpy(&f, &u, 4);
    return f;
}

static float orc_round_fp16(float f)
{
    uint32_t u;
    memcpy(&u, &f, 4);
    uint32_t sign = u & 0x80000000u;
    uint32_t absu = u & 0x7fffffffu;
    float r;
    if (absu >= 0x7f800000u)
    {
        return f; /* inf / nan unchanged */
    }
    if (absu >= 0x477ff000u)
    {
        /* >= 65520 rounds to infinity in binary16 */
        uint32_t inf = sign | 0x7f800000u;
        memcpy(&r, &inf, 4);
        return r;
    }
    if (absu < 0x38800000u)
    {
        /* below the smallest normal half (2^-14): quantise to multiples of 2^-24 */
        float a;
        memcpy(&a, &absu, 4);
        float q = a * 16777216.0f; /* exact scaling */
        q       = rintf(q);        /* FE_TONEAREST, ties to even */
        a       = q / 16777216.0f;
        uint32_t au;
        memcpy(&au, &a, 4);
        au |= sign;
        memcpy(&r, &au, 4);
        return r;
    }
    {
        uint32_t lsb = (absu >> 13) & 1u;
        absu += 0x0fffu + lsb;
        absu &= 0xffffe000u;
        absu |= sign;
        memcpy(&r, &absu, 4);
        return r;
    }
}

/* dtype codes for the float helpers: 0 = fp32 (no-op), 1 = fp16, 2 = bf16 */
static float orc_fptrunc(float f, int fdt)
{
    if (fdt == 1)
        return orc_round_fp16(f);
    if (fdt == 2)
        return orc_round_bf16(f);
    return f;
}

ORC_API void orc_fptrunc_array(const float* in, float* out, int64_t n, int fdt)
{
    for (int64_t i = 0; i < n; i++)
        out[i] = orc_fptrunc(in[i], fdt);
}

/* ------------------------------------------------------------------------- */
/* Attribute checks                                                           */
/* ------------------------------------------------------------------------- */

/* check_conv_attribute, src/ops/tensor_ops.cpp:120-226 (2-D case).
 * Returns 0 when legal, else a small positive code naming the failed rule. */
ORC_API int orc_check_conv2d_attribute(int IH, int IW, int OH, int OW, int KH, int KW, const int* pad,
                                       const int* stride, const int* dilation)
{
    for (int i = 0; i < 4; i++)
        if (pad[i] < 0)
            return 1;
    for (int i = 0; i < 2; i++)
        if (stride[i] < 1)
            return 2;
    for (int i = 0; i < 2; i++)
        if (dilation[i] < 1)
            return 3;
    int full_H = IH - 1 + pad[0] + pad[1] - (KH - 1) * dilation[0];
    int full_W = IW - 1 + pad[2] + pad[3] - (KW - 1) * dilation[1];
    if ((full_H % stride[0] != 0) || (full_W % stride[1] != 0))
        return 4;
    if ((OH != full_H / stride[0] + 1) || (OW != full_W / stride[1] + 1))
        return 5;
    return 0;
}

/* check_pool2d_attribute, src/ops/tensor_ops.cpp:28-117 */
ORC_API int orc_check_pool2d_attribute(int IH, int IW, int OH, int OW, const int* kernel, const int* pad,
                                       const int* stride)
{
    for (int i = 0; i < 4; i++)
        if (pad[i] < 0)
            return 1;
    for (int i = 0; i < 2; i++)
        if (kernel[i] < 1)
            return 2;
    for (int i = 0; i < 2; i++)
        if (stride[i] < 1)
            return 3;
    if (pad[0] >= kernel[0] || pad[1] >= kernel[0] || pad[2] >= kernel[1] || pad[3] >= kernel[1])
        return 4;
    int full_H = IH + pad[0] + pad[1] - kernel[0];
    int full_W = IW + pad[2] + pad[3] - kernel[1];
    if ((full_H % stride[0] != 0) || (full_W % stride[1] != 0))
        return 5;
    if ((OH != full_H / stride[0] + 1) || (OW != full_W / stride[1] + 1))
        return 6;
    return 0;
}

/* ------------------------------------------------------------------------- */
/* CONV2D  (OpConv2d::eval, src/ops/tensor_ops.cpp:723-882)                   */
/*   out = bias[oc or 0] + Out(sum over in-scope taps (in - in_zp)(w - w_zp)) */
/*   tap order ky -> kx -> ic (:836-865); out-of-scope taps skipped (:847-852)*/
/* ------------------------------------------------------------------------- */
#define ORC_CONV2D_BODY(TIN, TACC, TOUT, ABSFN, BOUNDS)                                                     \
    _Pragma("omp parallel for collapse(2) num_threads(nthreads) if (nthreads > 1)") for (int ob = 0;       \
                                                                                          ob < N; ob++)    \
    {                                                                                                       \
        for (int oy = 0; oy < OH; oy++)                                                                     \
        {                                                                                                   \
            for (int ox = 0; ox < OW; ox++)                                                                 \
            {                                                                                               \
                for (int oc = 0; oc < OC; oc++)                                                             \
                {                                                                                           \
                    TACC acc = 0;                                                                           \
                    for (int ky = 0; ky < KH; ky++)                                                         \
                    {                                                                                       \
                        int y = oy * stride[0] + ky * dilation[0] - pad[0];                                 \
                        for (int kx = 0; kx < KW; kx++)                                                     \
                        {                                                                                   \
                            int x = ox * stride[1] + kx * dilation[1] - pad[2];                             \
                            if (!((0 <= x && x < IW) && (0 <= y && y < IH)))                                \
                                continue;                                                                   \
                            const TIN* ip = in + (((int64_t)ob * IH + y) * IW + x) * IC;                    \
                            const TIN* wp = w + (((int64_t)oc * KH + ky) * KW + kx) * IC;                   \
                            for (int ic = 0; ic < IC; ic++)                                                 \
                            {                                                                               \
                                TACC a = (BOUNDS) ? (TACC)ABSFN(ip[ic]) : (TACC)ip[ic];                     \
                                TACC b = (BOUNDS) ? (TACC)ABSFN(wp[ic]) : (TACC)wp[ic];                     \
                                if ((BOUNDS) && !local_bound)                                               \
                                    a = (TACC)in_absmax;                                                    \
                                acc += (a - (TACC)in_zp) * (b - (TACC)w_zp);                                \
                            }                                                                               \
                        }                                                                                   \
                    }                                                                                       \
                    TOUT bv = bias[bias_n == 1 ? 0 : oc];                                                   \
                    if (BOUNDS)                                                                             \
                        bv = (TOUT)ABSFN(bv);                                                               \
                    out[(((int64_t)ob * OH + oy) * OW + ox) * OC + oc] = bv + (TOUT)acc;                    \
                }                                                                                           \
            }                                                                                               \
        }                                                                                                   \
    }

/* integer instantiation <INT8,INT8,INT32,INT32> (src/ops/tensor_ops.cpp:2224) */
ORC_API void orc_conv2d_i32(const int32_t* in, const int32_t* w, const int32_t* bias, int bias_n, int N, int IH,
                            int IW, int IC, int OC, int KH, int KW, int OH, int OW, const int* pad,
                            const int* stride, const int* dilation, int32_t in_zp, int32_t w_zp, int32_t* out,
                            int nthreads)
{
    const int local_bound   = 1;
    const int32_t in_absmax = 0;
    /* int32 arithmetic wraps like the two's-complement hardware the reference runs on */
    ORC_CONV2D_BODY(int32_t, uint32_t, uint32_t, abs, 0)
}

/* fp instantiations with an fp32 accumulator, <FP16,FP16,FP32,FP16>, <BF16,...>, <FP32,...>
 * (src/ops/tensor_ops.cpp:2220-2223): inputs are floats holding fp16/bf16/fp32 values, sequential
 * float accumulation, result left as float (not narrowed inside the op). */
ORC_API void orc_conv2d_f32(const float* in, const float* w, const float* bias, int bias_n, int N, int IH, int IW,
                            int IC, int OC, int KH, int KW, int OH, int OW, const int* pad, const int* stride,
                            const int* dilation, float* out, int nthreads)
{
    const float in_zp = 0, w_zp = 0, in_absmax = 0;
    const int local_bound = 1;
    ORC_CONV2D_BODY(float, float, float, fabsf, 0)
}

/* precise mode (all fp dtypes become FP64, include/dtype.h:124-152) and its bounds variant
 * (abs of operands, src/ops/tensor_ops.cpp:790-802). */
ORC_API void orc_conv2d_f64(const double* in, const double* w, const double* bias, int bias_n, int N, int IH, int IW,
                            int IC, int OC, int KH, int KW, int OH, int OW, const int* pad, const int* stride,
                            const int* dilation, int bounds_mode, int local_bound, double* out, int nthreads)
{
    const double in_zp = 0, w_zp = 0;
    double in_absmax = 0;
    if (bounds_mode && !local_bound)
    {
        int64_t n = (int64_t)N * IH * IW * IC;
        for (int64_t i = 0; i < n; i++)
            if (fabs(in[i]) > in_absmax)
                in_absmax = fabs(in[i]);
    }
    if (bounds_mode)
    {
        ORC_CONV2D_BODY(double, double, double, fabs, 1)
    }
    else
    {
        ORC_CONV2D_BODY(double, double, double, fabs, 0)
    }
}

/* ------------------------------------------------------------------------- */
/* CONV3D (OpConv3d::eval, src/ops/tensor_ops.cpp:934-1120)                    */
/*   input [N,ID,IH,IW,IC], weights [OC,KD,KH,KW,IC], pad = (d0,d1,t,b,l,r),   */
/*   stride / dilation = (d,y,x); taps outside the input are skipped (:1077);  */
/*   order kd -> ky -> kx -> ic, sequential (:1060-1099); bias added last.     */
/* ------------------------------------------------------------------------- */

/* check_conv_attribute with conv_dimension 3 (src/ops/tensor_ops.cpp:120-226) */
ORC_API int orc_check_conv3d_attribute(int ID, int IH, int IW, int OD, int OH, int OW, int KD, int KH, int KW,
                                       const int* pad, const int* stride, const int* dilation)
{
    for (int i = 0; i < 6; i++)
        if (pad[i] < 0)
            return 1;
    for (int i = 0; i < 3; i++)
        if (stride[i] < 1)
            return 2;
    for (int i = 0; i < 3; i++)
        if (dilation[i] < 1)
            return 3;
    int full_D = ID - 1 + pad[0] + pad[1] - (KD - 1) * dilation[0];
    int full_H = IH - 1 + pad[2] + pad[3] - (KH - 1) * dilation[1];
    int full_W = IW - 1 + pad[4] + pad[5] - (KW - 1) * dilation[2];
    if ((full_D % stride[0] != 0) || (full_H % stride[1] != 0) || (full_W % stride[2] != 0))
        return 4;
    if ((OD != full_D / stride[0] + 1) || (OH != full_H / stride[1] + 1) || (OW != full_W / stride[2] + 1))
        return 5;
    return 0;
}

#define ORC_CONV3D_BODY(TIN, TACC, TOUT, ABSFN, BOUNDS)                                                         \
    _Pragma("omp parallel for collapse(2) num_threads(nthreads) if (nthreads > 1)") for (int ob = 0; ob < N; ob++) \
    {                                                                                                           \
        for (int od = 0; od < OD; od++)                                                                         \
        {                                                                                                       \
            for (int oy = 0; oy < OH; oy++)                                                                     \
                for (int ox = 0; ox < OW; ox++)                                                                 \
                    for (int oc = 0; oc < OC; oc++)                                                             \
                    {                                                                                           \
                        TACC acc = 0;                                                                           \
                        for (int kd = 0; kd < KD; kd++)                                                         \
                        {                                                                                       \
                            int d = od * stride[0] + kd * dilation[0] - pad[0];                                 \
                            for (int ky = 0; ky < KH; ky++)                                                     \
                            {                                                                                   \
                                int y = oy * stride[1] + ky * dilation[1] - pad[2];                             \
                                for (int kx = 0; kx < KW; kx++)                                                 \
                                {                                                                               \
                                    int x = ox * stride[2] + kx * dilation[2] - pad[4];                         \
                                    if (!((0 <= x && x < IW) && (0 <= y && y < IH) && (0 <= d && d < ID)))      \
                                        continue;                                                               \
                                    const TIN* ip = in + ((((int64_t)ob * ID + d) * IH + y) * IW + x) * IC;     \
                                    const TIN* wp = w + ((((int64_t)oc * KD + kd) * KH + ky) * KW + kx) * IC;   \
                                    for (int ic = 0; ic < IC; ic++)                                             \
                                    {                                                                           \
                                        TACC a = (BOUNDS) ? (TACC)ABSFN(ip[ic]) : (TACC)ip[ic];                 \
                                        TACC b = (BOUNDS) ? (TACC)ABSFN(wp[ic]) : (TACC)wp[ic];                 \
                                        if ((BOUNDS) && !local_bound)                                           \
                                            a = (TACC)in_absmax;                                                \
                                        acc += (a - (TACC)in_zp) * (b - (TACC)w_zp);                            \
                                    }                                                                           \
                                }                                                                               \
                            }                                                                                   \
                        }                                                                                       \
                        TOUT bv = bias[bias_n == 1 ? 0 : oc];                                                   \
                        if (BOUNDS)                                                                             \
                            bv = (TOUT)ABSFN(bv);                                                               \
                        out[((((int64_t)ob * OD + od) * OH + oy) * OW + ox) * OC + oc] = bv + (TOUT)acc;        \
                    }                                                                                           \
        }                                                                                                       \
    }

/* dims = {N, ID, IH, IW, IC, OC, KD, KH, KW, OD, OH, OW} */
#define ORC_CONV3D_DIMS                                                                                          \
    const int N = dims[0], ID = dims[1], IH = dims[2], IW = dims[3], IC = dims[4], OC = dims[5], KD = dims[6],   \
              KH = dims[7], KW = dims[8], OD = dims[9], OH = dims[10], OW = dims[11];

/* integer instantiation <INT8,INT8,INT32,INT32> (src/ops/tensor_ops.cpp:2235) */
ORC_API void orc_conv3d_i32(const int32_t* in, const int32_t* w, const int32_t* bias, int bias_n, const int* dims,
                            const int* pad, const int* stride, const int* dilation, int32_t in_zp, int32_t w_zp,
                            int32_t* out, int nthreads)
{
    ORC_CONV3D_DIMS
    const int local_bound   = 1;
    const int32_t in_absmax = 0;
    ORC_CONV3D_BODY(int32_t, uint32_t, uint32_t, abs, 0)
}

/* floating instantiations with an fp32 accumulator: sequential float accumulation, result left as float */
ORC_API void orc_conv3d_f32(const float* in, const float* w, const float* bias, int bias_n, const int* dims,
                            const int* pad, const int* stride, const int* dilation, float* out, int nthreads)
{
    ORC_CONV3D_DIMS
    const float in_zp = 0, w_zp = 0, in_absmax = 0;
    const int local_bound = 1;
    ORC_CONV3D_BODY(float, float, float, fabsf, 0)
}

/* precise mode and its bounds variant (abs of operands, src/ops/tensor_ops.cpp:1015-1027) */
ORC_API void orc_conv3d_f64(const double* in, const double* w, const double* bias, int bias_n, const int* dims,
                            const int* pad, const int* stride, const int* dilation, int bounds_mode, int local_bound,
                            double* out, int nthreads)
{
    ORC_CONV3D_DIMS
    const double in_zp = 0, w_zp = 0;
    double in_absmax = 0;
    if (bounds_mode && !local_bound)
    {
        int64_t n = (int64_t)N * ID * IH * IW * IC;
        for (int64_t i = 0; i < n; i++)
            if (fabs(in[i]) > in_absmax)
                in_absmax = fabs(in[i]);
    }
    if (bounds_mode)
    {
        ORC_CONV3D_BODY(double, double, double, fabs, 1)
    }
    else
    {
        ORC_CONV3D_BODY(double, double, double, fabs, 0)
    }
}

/* ------------------------------------------------------------------------- */
/* DEPTHWISE_CONV2D (OpDepthwiseConv2d::eval, src/ops/tensor_ops.cpp:1172-1334)*/
/*   weights [KH,KW,C,M]; output channel c*M+m (:1320); order ky -> kx         */
/* ------------------------------------------------------------------------- */
#define ORC_DW_BODY(TIN, TACC, TOUT, ABSFN, BOUNDS)                                                          \
    _Pragma("omp parallel for collapse(2) num_threads(nthreads) if (nthreads > 1)") for (int ob = 0;        \
                                                                                          ob < N; ob++)     \
    {                                                                                                        \
        for (int oy = 0; oy < OH; oy++)                                                                      \
        {                                                                                                    \
            for (int ox = 0; ox < OW; ox++)                                                                  \
            {                                                                                                \
                for (int ic = 0; ic < C; ic++)                                                               \
                {                                                                                            \
                    for (int km = 0; km < M; km++)                                                           \
                    {                                                                                        \
                        TACC acc = 0;                                                                        \
                        int iy   = oy * stride[0] - pad[0];                                                  \
                        int ix   = ox * stride[1] - pad[2];                                                  \
                        for (int ky = 0; ky < KH; ky++)                                                      \
                        {                                                                                    \
                            for (int kx = 0; kx < KW; kx++)                                                  \
                            {                                                                                \
                                int y = iy + ky * dilation[0];                                               \
                                int x = ix + kx * dilation[1];                                               \
                                if (!((0 <= y && y < IH) && (0 <= x && x < IW)))                             \
                                    continue;                                                                \
                                TIN iv = in[(((int64_t)ob * IH + y) * IW + x) * C + ic];                     \
                                TIN wv = w[(((int64_t)ky * KW + kx) * C + ic) * M + km];                     \
                                TACC a = (BOUNDS) ? (TACC)ABSFN(iv) : (TACC)iv;                              \
                                TACC b = (BOUNDS) ? (TACC)ABSFN(wv) : (TACC)wv;                              \
                                if ((BOUNDS) && !local_bound)                                                \
                                    a = (TACC)in_absmax;                                                     \
                                acc += (a - (TACC)in_zp) * (b - (TACC)w_zp);                                 \
                            }                                                                                \
                        }                                                                                    \
                        int oc  = ic * M + km;                                                               \
                        TOUT bv = bias[bias_n == 1 ? 0 : oc];                                                \
                        if (BOUNDS)                                                                          \
                            bv = (TOUT)ABSFN(bv);                                                            \
                        out[(((int64_t)ob * OH + oy) * OW + ox) * (C * M) + oc] = bv + (TOUT)acc;            \
                    }                                                                                        \
                }                                                                                            \
            }                                                                                                \
        }                                                                                                    \
    }

ORC_API void orc_depthwise_conv2d_i32(const int32_t* in, const int32_t* w, const int32_t* bias, int bias_n, int N,
                                      int IH, int IW, int C, int M, int KH, int KW, int OH, int OW, const int* pad,
                                      const int* stride, const int* dilation, int32_t in_zp, int32_t w_zp,
                                      int32_t* out, int nthreads)
{
    const int local_bound   = 1;
    const int32_t in_absmax = 0;
    ORC_DW_BODY(int32_t, uint32_t, uint32_t, abs, 0)
}

ORC_API void orc_depthwise_conv2d_f32(const float* in, const float* w, const float* bias, int bias_n, int N, int IH,
                                      int IW, int C, int M, int KH, int KW, int OH, int OW, const int* pad,
                                      const int* stride, const int* dilation, float* out, int nthreads)
{
    const float in_zp = 0, w_zp = 0, in_absmax = 0;
    const int local_bound = 1;
    ORC_DW_BODY(float, float, float, fabsf, 0)
}

ORC_API void orc_depthwise_conv2d_f64(const double* in, const double* w, const double* bias, int bias_n, int N,
                                      int IH, int IW, int C, int M, int KH, int KW, int OH, int OW, const int* pad,
                                      const int* stride, const int* dilation, int bounds_mode, int local_bound,
                                      double* out, int nthreads)
{
    const double in_zp = 0, w_zp = 0;
    double in_absmax = 0;
    if (bounds_mode && !local_bound)
    {
        int64_t n = (int64_t)N * IH * IW * C;
        for (int64_t i = 0; i < n; i++)
            if (fabs(in[i]) > in_absmax)
                in_absmax = fabs(in[i]);
    }
    if (bounds_mode)
    {
        ORC_DW_BODY(double, double, double, fabs, 1)
    }
    else
    {
        ORC_DW_BODY(double, double, double, fabs, 0)
    }
}

/* ------------------------------------------------------------------------- */
/* TRANSPOSE_CONV2D (OpTransposeConv2d::eval, src/ops/tensor_ops.cpp:2059-2197)*/
/*   per output (oy, ox): iy = oy - out_pad_top, y = iy - ky; the tap is in     */
/*   scope when 0 <= y < IH*stride_y and y % stride_y == 0 (same for x), and    */
/*   then reads in(y/stride_y, x/stride_x) (:2148-2171); tap order ky -> kx ->  */
/*   ic; out = (Out)acc + bias[oc or 0] (:2176-2177); weights OHWI, not flipped.*/
/*   The reference's own tests hold no known-answer vector for this operator:   */
/*   the restatement is pinned through its identity with the pinned CONV2D      */
/*   restatement above (zero-stuffed input, mirrored kernel) and a hand case.   */
/* ------------------------------------------------------------------------- */
/* returns 0 when OpTransposeConv2d::checkTensorAttributes (:1982-2056) accepts the attributes */
ORC_API int orc_check_transpose_conv2d_attribute(int IH, int IW, int OH, int OW, int KH, int KW, const int* out_pad,
                                                 const int* stride)
{
    if (stride[0] < 1 || stride[1] < 1)
        return 1;
    if (out_pad[0] <= -KH || out_pad[1] <= -KH || out_pad[2] <= -KW || out_pad[3] <= -KW)
        return 2;
    if (OH != (IH - 1) * stride[0] + out_pad[0] + out_pad[1] + KH)
        return 3;
    if (OW != (IW - 1) * stride[1] + out_pad[2] + out_pad[3] + KW)
        return 3;
    return 0;
}

#define ORC_TCONV_BODY(TIN, TACC, TOUT)                                                                      \
    _Pragma("omp parallel for collapse(2) num_threads(nthreads) if (nthreads > 1)") for (int ob = 0;        \
                                                                                          ob < N; ob++)     \
    {                                                                                                        \
        for (int oy = 0; oy < OH; oy++)                                                                      \
        {                                                                                                    \
            for (int ox = 0; ox < OW; ox++)                                                                  \
            {                                                                                                \
                int iy = oy - out_pad[0];                                                                    \
                int ix = ox - out_pad[2];                                                                    \
                for (int oc = 0; oc < OC; oc++)                                                              \
                {                                                                                            \
                    TACC acc = 0;                                                                            \
                    for (int ky = 0; ky < KH; ky++)                                                          \
                    {                                                                                        \
                        for (int kx = 0; kx < KW; kx++)                                                      \
                        {                                                                                    \
                            int y = iy - ky;                                                                 \
                            int x = ix - kx;                                                                 \
                            int in_scope = (0 <= y && y < IH * stride[0]) && (0 <= x && x < IW * stride[1]) && \
                                           (y % stride[0] == 0) && (x % stride[1] == 0);                     \
                            if (!in_scope)                                                                   \
                                continue;                                                                    \
                            const TIN* ip = in + (((int64_t)ob * IH + y / stride[0]) * IW + x / stride[1]) * IC; \
                            const TIN* wp = w + (((int64_t)oc * KH + ky) * KW + kx) * IC;                    \
                            for (int ic = 0; ic < IC; ic++)                                                  \
                                acc += ((TACC)ip[ic] - (TACC)in_zp) * ((TACC)wp[ic] - (TACC)w_zp);          \
                        }                                                                                    \
                    }                                                                                        \
                    out[(((int64_t)ob * OH + oy) * OW + ox) * OC + oc] = (TOUT)acc + bias[bias_n == 1 ? 0 : oc]; \
                }                                                                                            \
            }                                                                                                \
        }                                                                                                    \
    }

/* integer instantiation <INT8,INT8,INT32,INT32> (src/ops/tensor_ops.cpp:2290) */
ORC_API void orc_transpose_conv2d_i32(const int32_t* in, const int32_t* w, const int32_t* bias, int bias_n, int N,
                                      int IH, int IW, int IC, int OC, int KH, int KW, int OH, int OW,
                                      const int* out_pad, const int* stride, int32_t in_zp, int32_t w_zp,
                                      int32_t* out, int nthreads)
{
    ORC_TCONV_BODY(int32_t, uint32_t, uint32_t)
}

/* floating instantiations with an fp32 accumulator (src/ops/tensor_ops.cpp:2286-2288) */
ORC_API void orc_transpose_conv2d_f32(const float* in, const float* w, const float* bias, int bias_n, int N, int IH,
                                      int IW, int IC, int OC, int KH, int KW, int OH, int OW, const int* out_pad,
                                      const int* stride, float* out, int nthreads)
{
    const float in_zp = 0, w_zp = 0;
    ORC_TCONV_BODY(float, float, float)
}

/* precise mode (all floating dtypes become FP64, include/dtype.h:124-152) */
ORC_API void orc_transpose_conv2d_f64(const double* in, const double* w, const double* bias, int bias_n, int N,
                                      int IH, int IW, int IC, int OC, int KH, int KW, int OH, int OW,
                                      const int* out_pad, const int* stride, double* out, int nthreads)
{
    const double in_zp = 0, w_zp = 0;
    ORC_TCONV_BODY(double, double, double)
}

/* ------------------------------------------------------------------------- */
/* MATMUL (OpMatMul::eval, src/ops/tensor_ops.cpp:1423-1492)                  */
/*   per batch n: out[n] = (A[n] - a_zp) x (B[n] - b_zp); A [N,H,C], B [N,C,W]*/
/*   The reference hands the product to Eigen's contraction (:1472); integer   */
/*   results do not depend on summation order.  Loop order here is h, c, w so  */
/*   the inner loop is unit-stride over both B and the output row.             */
/* ------------------------------------------------------------------------- */
#define ORC_MATMUL_BODY(TIN, TACC, ABSFN, BOUNDS)                                                           \
    _Pragma("omp parallel for collapse(2) num_threads(nthreads) if (nthreads > 1)") for (int n = 0; n < N;  \
                                                                                          n++)              \
    {                                                                                                       \
        for (int h = 0; h < H; h++)                                                                         \
        {                                                                                                   \
            TACC* orow = (TACC*)(out + ((int64_t)n * H + h) * W);                                           \
            for (int wv = 0; wv < W; wv++)                                                                  \
                orow[wv] = 0;                                                                               \
            for (int c = 0; c < C; c++)                                                                     \
            {                                                                                               \
                TIN av       = a[((int64_t)n * H + h) * C + c];                                             \
                TACC aval    = ((BOUNDS) ? (TACC)ABSFN(av) : (TACC)av) - (TACC)a_zp;                        \
                const TIN* br = b + ((int64_t)n * C + c) * W;                                               \
                for (int wv = 0; wv < W; wv++)                                                              \
                {                                                                                           \
                    TACC bval = ((BOUNDS) ? (TACC)ABSFN(br[wv]) : (TACC)br[wv]) - (TACC)b_zp;               \
                    orow[wv] += aval * bval;                                                                \
                }                                                                                           \
            }                                                                                               \
        }                                                                                                   \
    }

ORC_API void orc_matmul_i32(const int32_t* a, const int32_t* b, int N, int H, int C, int W, int32_t a_zp,
                            int32_t b_zp, int32_t* out, int nthreads)
{
    ORC_MATMUL_BODY(int32_t, uint32_t, abs, 0)
}

ORC_API void orc_matmul_f32(const float* a, const float* b, int N, int H, int C, int W, float* out, int nthreads)
{
    const float a_zp = 0, b_zp = 0;
    ORC_MATMUL_BODY(float, float, fabsf, 0)
}

ORC_API void orc_matmul_f64(const double* a, const double* b, int N, int H, int C, int W, int bounds_mode,
                            double* out, int nthreads)
{
    const double a_zp = 0, b_zp = 0;
    if (bounds_mode)
    {
        ORC_MATMUL_BODY(double, double, fabs, 1)
    }
    else
    {
        ORC_MATMUL_BODY(double, double, fabs, 0)
    }
}

/* ------------------------------------------------------------------------- */
/* RESCALE                                                                    */
/* ------------------------------------------------------------------------- */

/* QuantUtil::apply_scale_32, src/quant_util.h:45-84.  Returns 0 and writes *res, or 1 when one of the
 * reference's range checks (which it turns into REQUIRE failures) is violated. */
static int apply_scale_32_impl(int32_t value, int32_t multiplier, int32_t shift, int double_round, int32_t* res)
{
    if (multiplier < 0)
        return 1;
    if (shift < 2 || shift > 62)
        return 1;
    int64_t low_val  = -((int64_t)1 << (shift - 1));
    int64_t high_val = (int64_t)1 << (shift - 1);
    if (value < low_val || value >= high_val)
        return 1;
    int64_t round = (int64_t)1 << (shift - 1);
    if (double_round)
    {
        if (shift > 31 && value >= 0)
            round += ((int64_t)1 << 30);
        if (shift > 31 && value < 0)
            round -= ((int64_t)1 << 30);
    }
    int64_t result = (int64_t)value * multiplier + round;
    result         = result >> shift;
    if (result < -((int64_t)1 << 31) || result >= ((int64_t)1 << 31))
        return 1;
    *res = (int32_t)result;
    return 0;
}

/* QuantUtil::apply_scale_16, src/quant_util.h:86-108 */
static int apply_scale_16_impl(int64_t value, int16_t multiplier, int32_t shift, int32_t* res)
{
    if (multiplier < 0)
        return 1;
    if (shift < 2 || shift > 62)
        return 1;
    int64_t round  = (int64_t)1 << (shift - 1);
    int64_t result = value * (int64_t)multiplier + round;
    result         = result >> shift;
    if (result < -((int64_t)1 << 31) || result >= ((int64_t)1 << 31))
        return 1;
    *res = (int32_t)result;
    return 0;
}

/* exported for known-answer tests of the scaling primitive */
ORC_API int orc_apply_scale_32(int32_t value, int32_t multiplier, int32_t shift, int double_round, int32_t* res)
{
    return apply_scale_32_impl(value, multiplier, shift, double_round, res);
}

/* value_extend64_impl, src/ops/type_conversion.cpp:183-221 (8/16/32-bit cases) */
static int64_t orc_value_extend64(int32_t val, int bits, int is_unsigned)
{
    switch (bits)
    {
        case 8:
            return is_unsigned ? (int64_t)(uint8_t)(val & 0xFF) : (int64_t)(int8_t)(val & 0xFF);
        case 16:
            return is_unsigned ? (int64_t)(uint16_t)(val & 0xFFFF) : (int64_t)(int16_t)(val & 0xFFFF);
        default:
            return is_unsigned ? (int64_t)(uint32_t)val : (int64_t)val;
    }
}

/* OpRescale::eval, src/ops/type_conversion.cpp:223-422, SINGLE_ROUND / DOUBLE_ROUND modes.
 *   in/out: [outer, C] int32 containers.  multiplier/shift: length C when per_channel else 1.
 *   rounding_mode: 0 = SINGLE_ROUND, 1 = DOUBLE_ROUND, 2 = INEXACT_ROUND (fp32 maths, :318-323).
 * Returns ORC_VALID, ORC_UNPREDICTABLE (a REQUIRE failed; output of that element left 0) or
 * ORC_ERROR (zero-point / attribute ERROR_IF, :118-132, :248-255). */
ORC_API int orc_rescale(const int32_t* in, int64_t outer, int C, const int32_t* multiplier, const int32_t* shift,
                        int per_channel, int scale32, int rounding_mode, int32_t input_zp, int32_t output_zp,
                        int in_bits, int out_bits, int input_unsigned, int output_unsigned, int32_t* out)
{
    const int double_round  = (rounding_mode == 1);
    const int inexact_round = (rounding_mode == 2);
    if (rounding_mode < 0 || rounding_mode > 2)
        return ORC_ERROR;
    if (!scale32 && double_round)
        return ORC_ERROR;
    if (input_unsigned && output_unsigned)
        return ORC_ERROR;
    if ((in_bits == 32 && input_unsigned) || (out_bits == 32 && output_unsigned))
        return ORC_ERROR;

    int64_t output_zp_extended = orc_value_extend64(output_zp, out_bits, output_unsigned);
    int64_t input_zp_extended  = orc_value_extend64(input_zp, in_bits, input_unsigned);
    if (in_bits != 8 && !(in_bits == 16 && input_unsigned) && input_zp_extended != 0)
        return ORC_ERROR;
    if (out_bits != 8 && !(out_bits == 16 && output_unsigned) && output_zp_extended != 0)
        return ORC_ERROR;
    if (in_bits == 16 && input_unsigned && input_zp_extended != 0 && input_zp_extended != 32768)
        return ORC_ERROR;
    if (out_bits == 16 && output_unsigned && output_zp_extended != 0 && output_zp_extended != 32768)
        return ORC_ERROR;

    /* clip ranges: QMin_s/QMax_s and QMin_u/QMax_u of the output width (src/arith_util.h:263-328) */
    int64_t qmin, qmax;
    if (output_unsigned)
    {
        qmin = 0;
        qmax = (out_bits == 8) ? 255 : (out_bits == 16) ? 65535 : (int64_t)2147483647; /* capped at int32 max */
    }
    else
    {
        qmin = -((int64_t)1 << (out_bits - 1));
        qmax = ((int64_t)1 << (out_bits - 1)) - 1;
    }

    int status = ORC_VALID;
    for (int64_t j = 0; j < outer; j++)
    {
        for (int c = 0; c < C; c++)
        {
            int32_t m   = multiplier[per_channel ? c : 0];
            int32_t s   = shift[per_channel ? c : 0];
            int64_t v64 = orc_value_extend64(in[j * C + c], in_bits, input_unsigned) - input_zp_extended;
            int32_t scaled;
            int bad = 0;
            if (!inexact_round)
            {
                if (scale32)
                    bad = apply_scale_32_impl((int32_t)v64, m, s, double_round, &scaled);
                else
                    bad = apply_scale_16_impl(v64, (int16_t)m, s, &scaled);
            }
            else
            {
                float res_f32 = (float)v64 * (float)m * exp2f((float)(-s));
                scaled        = (int32_t)rintf(res_f32);
            }
            if (bad)
            {
                status          = ORC_UNPREDICTABLE;
                out[j * C + c] = 0;
                continue;
            }
            int64_t r = (int64_t)scaled + output_zp_extended;
            if (r > 2147483647LL || r < -2147483648LL)
            {
                status          = ORC_UNPREDICTABLE;
                out[j * C + c] = 0;
                continue;
            }
            if (r < qmin)
                r = qmin;
            if (r > qmax)
                r = qmax;
            out[j * C + c] = (int32_t)r;
        }
    }
    return status;
}

/* ------------------------------------------------------------------------- */
/* CLAMP (OpClamp::register_fcn, src/ops/activation_funcs.cpp:27-128;          */
/*        applyClip, src/arith_util.h:389-413)                                 */
/* ------------------------------------------------------------------------- */
ORC_API int orc_clamp_i32(const int32_t* in, int64_t n, int32_t min_val, int32_t max_val, int32_t* out)
{
    if (max_val < min_val)
        return ORC_ERROR;
    for (int64_t i = 0; i < n; i++)
    {
        int32_t v = in[i];
        v         = (v >= min_val) ? v : min_val;
        v         = (v < max_val) ? v : max_val;
        out[i]    = v;
    }
    return ORC_VALID;
}

/* fp CLAMP: clip, then fpTrunc to the storage dtype (:105-111).  nan_ignore selects NanPropagationMode_IGNORE:
 * a NaN input then takes the other operand of max/min (src/arith_util.h:340-386). */
ORC_API int orc_clamp_f32(const float* in, int64_t n, float min_val, float max_val, int fdt, int nan_ignore,
                          float* out)
{
    if (isnan(min_val) || isnan(max_val))
        return ORC_ERROR;
    if (max_val < min_val)
        return ORC_ERROR;
    for (int64_t i = 0; i < n; i++)
    {
        float v = in[i];
        if (isnan(v))
            v = nan_ignore ? min_val : NAN;
        else
            v = (v >= min_val) ? v : min_val;
        if (!isnan(v))
            v = (v < max_val) ? v : max_val;
        out[i] = orc_fptrunc(v, fdt);
    }
    return ORC_VALID;
}

ORC_API int orc_clamp_f64(const double* in, int64_t n, double min_val, double max_val, double* out)
{
    if (max_val < min_val)
        return ORC_ERROR;
    for (int64_t i = 0; i < n; i++)
    {
        double v = in[i];
        if (!isnan(v))
        {
            v = (v >= min_val) ? v : min_val;
            v = (v < max_val) ? v : max_val;
        }
        out[i] = v;
    }
    return ORC_VALID;
}

/* ------------------------------------------------------------------------- */
/* ADD (OpAdd::register_fcn, src/ops/ewise_binary.cpp:144-173; broadcast :81-111)*/
/* Rank-4-or-less tensors, size-1 dimensions of either operand broadcast.       */
/* ------------------------------------------------------------------------- */
static int orc_bcast_shape(int rank, const int* a_shape, const int* b_shape, const int* o_shape)
{
    for (int i = 0; i < rank; i++)
    {
        int cs = a_shape[i];
        if (cs == 1)
            cs = b_shape[i];
        else if (b_shape[i] != 1 && b_shape[i] != cs)
            return 1;
        if (cs != o_shape[i])
            return 1;
    }
    return 0;
}

#define ORC_ADD_LOOP(EXPR)                                                                                  \
    int as[6] = { 1, 1, 1, 1, 1, 1 }, bs[6] = { 1, 1, 1, 1, 1, 1 }, os[6] = { 1, 1, 1, 1, 1, 1 };           \
    for (int i = 0; i < rank; i++)                                                                          \
    {                                                                                                       \
        as[6 - rank + i] = a_shape[i];                                                                      \
        bs[6 - rank + i] = b_shape[i];                                                                      \
        os[6 - rank + i] = o_shape[i];                                                                      \
    }                                                                                                       \
    int64_t total = 1;                                                                                      \
    for (int i = 0; i < 6; i++)                                                                             \
        total *= os[i];                                                                                     \
    for (int64_t idx = 0; idx < total; idx++)                                                               \
    {                                                                                                       \
        int64_t rem = idx, ai = 0, bi = 0, am = 1, bm = 1;                                                  \
        for (int d = 5; d >= 0; d--)                                                                        \
        {                                                                                                   \
            int64_t c = rem % os[d];                                                                        \
            rem /= os[d];                                                                                   \
            if (as[d] != 1)                                                                                 \
                ai += c * am;                                                                               \
            if (bs[d] != 1)                                                                                 \
                bi += c * bm;                                                                               \
            am *= as[d];                                                                                    \
            bm *= bs[d];                                                                                    \
        }                                                                                                   \
        EXPR;                                                                                               \
    }

/* INT32 ADD.  The reference forms the sum in 32 bits before widening (:150), so the stored value is the
 * wrapped sum; the REQUIRE that the mathematical sum fits int32 is reported as ORC_UNPREDICTABLE. */
ORC_API int orc_add_i32(const int32_t* a, const int32_t* b, int rank, const int* a_shape, const int* b_shape,
                        const int* o_shape, int32_t* out)
{
    if (rank > 6 || orc_bcast_shape(rank, a_shape, b_shape, o_shape))
        return ORC_ERROR;
    int status = ORC_VALID;
    ORC_ADD_LOOP({
        int64_t s = (int64_t)a[ai] + (int64_t)b[bi];
        if (s > 2147483647LL || s < -2147483648LL)
            status = ORC_UNPREDICTABLE;
        out[idx] = (int32_t)(uint32_t)((uint32_t)a[ai] + (uint32_t)b[bi]);
    })
    return status;
}

/* fp ADD: fpTrunc<Out>(a + b) (:160-163) */
ORC_API int orc_add_f32(const float* a, const float* b, int rank, const int* a_shape, const int* b_shape,
                        const int* o_shape, int fdt, float* out)
{
    if (rank > 6 || orc_bcast_shape(rank, a_shape, b_shape, o_shape))
        return ORC_ERROR;
    ORC_ADD_LOOP({ out[idx] = orc_fptrunc(a[ai] + b[bi], fdt); })
    return ORC_VALID;
}

ORC_API int orc_add_f64(const double* a, const double* b, int rank, const int* a_shape, const int* b_shape,
                        const int* o_shape, double* out)
{
    if (rank > 6 || orc_bcast_shape(rank, a_shape, b_shape, o_shape))
        return ORC_ERROR;
    ORC_ADD_LOOP({ out[idx] = a[ai] + b[bi]; })
    return ORC_VALID;
}

/* ------------------------------------------------------------------------- */
/* MAX_POOL2D (OpMaxPool2d::eval, src/ops/tensor_ops.cpp:1545-1641)            */
/*   padding value = lowest of the dtype (src/arith_util.h:425-432), max over   */
/*   the kernel window.  `lowest` is passed in (-128 for int8, -32768 int16).   */
/* ------------------------------------------------------------------------- */
ORC_API void orc_max_pool2d_i32(const int32_t* in, int N, int IH, int IW, int C, int OH, int OW, const int* kernel,
                                const int* pad, const int* stride, int32_t lowest, int32_t* out)
{
    for (int n = 0; n < N; n++)
        for (int oy = 0; oy < OH; oy++)
            for (int ox = 0; ox < OW; ox++)
                for (int c = 0; c < C; c++)
                {
                    int32_t m = lowest;
                    for (int ky = 0; ky < kernel[0]; ky++)
                        for (int kx = 0; kx < kernel[1]; kx++)
                        {
                            int y     = oy * stride[0] - pad[0] + ky;
                            int x     = ox * stride[1] - pad[2] + kx;
                            int32_t v = lowest;
                            if (0 <= y && y < IH && 0 <= x && x < IW)
                                v = in[(((int64_t)n * IH + y) * IW + x) * C + c];
                            m = (m >= v) ? m : v;
                        }
                    out[(((int64_t)n * OH + oy) * OW + ox) * C + c] = m;
                }
}

/* fp MAX_POOL2D, NaN-propagating mode: padding is the lowest finite value of the dtype */
ORC_API void orc_max_pool2d_f32(const float* in, int N, int IH, int IW, int C, int OH, int OW, const int* kernel,
                                const int* pad, const int* stride, float lowest, float* out)
{
    for (int n = 0; n < N; n++)
        for (int oy = 0; oy < OH; oy++)
            for (int ox = 0; ox < OW; ox++)
                for (int c = 0; c < C; c++)
                {
                    float m = lowest;
                    for (int ky = 0; ky < kernel[0]; ky++)
                        for (int kx = 0; kx < kernel[1]; kx++)
                        {
                            int y   = oy * stride[0] - pad[0] + ky;
                            int x   = ox * stride[1] - pad[2] + kx;
                            float v = lowest;
                            if (0 <= y && y < IH && 0 <= x && x < IW)
                                v = in[(((int64_t)n * IH + y) * IW + x) * C + c];
                            if (isnan(m) || isnan(v))
                                m = NAN;
                            else
                                m = (m >= v) ? m : v;
                        }
                    out[(((int64_t)n * OH + oy) * OW + ox) * C + c] = m;
                }
}

/* ------------------------------------------------------------------------- */
/* AVG_POOL2D, integer path (OpAvgPool2d::eval, src/ops/tensor_ops.cpp:542-671;*/
/*   QuantUtil::reciprocal_scale, src/quant_util.h:32-43)                       */
/* ------------------------------------------------------------------------- */
ORC_API void orc_reciprocal_scale(int32_t value, int32_t* multiplier, int32_t* shift)
{
    uint32_t v   = (uint32_t)value;
    int32_t k    = (v - 1 == 0) ? 0 : 32 - __builtin_clz(v - 1);
    int64_t num  = (((int64_t)1 << 30) + 1) << k;
    *multiplier  = (int32_t)(num / value);
    *shift       = 30 + k;
}

ORC_API int orc_avg_pool2d_i32(const int32_t* in, int N, int IH, int IW, int C, int OH, int OW, const int* kernel,
                               const int* pad, const int* stride, int32_t input_zp, int32_t output_zp, int32_t qmin,
                               int32_t qmax, int32_t* out)
{
    int status = ORC_VALID;
    for (int n = 0; n < N; n++)
        for (int oy = 0; oy < OH; oy++)
            for (int ox = 0; ox < OW; ox++)
                for (int c = 0; c < C; c++)
                {
                    int32_t acc = 0;
                    int count   = 0;
                    for (int ky = 0; ky < kernel[0]; ky++)
                        for (int kx = 0; kx < kernel[1]; kx++)
                        {
                            int y = oy * stride[0] - pad[0] + ky;
                            int x = ox * stride[1] - pad[2] + kx;
                            if (0 <= y && y < IH && 0 <= x && x < IW)
                            {
                                acc = (int32_t)((uint32_t)acc +
                                                (uint32_t)(in[(((int64_t)n * IH + y) * IW + x) * C + c] - input_zp));
                                count++;
                            }
                        }
                    int32_t mult, shift, r;
                    orc_reciprocal_scale(count, &mult, &shift);
                    if (apply_scale_32_impl(acc, mult, shift, 0, &r))
                    {
                        status = ORC_UNPREDICTABLE;
                        r      = 0;
                    }
                    r = (int32_t)((uint32_t)r + (uint32_t)output_zp);
                    r = r > qmin ? r : qmin;
                    r = r < qmax ? r : qmax;
                    out[(((int64_t)n * OH + oy) * OW + ox) * C + c] = r;
                }
    return status;
}

/* fp AVG_POOL2D: acc / count in the accumulator type (:661-664) */
ORC_API void orc_avg_pool2d_f32(const float* in, int N, int IH, int IW, int C, int OH, int OW, const int* kernel,
                                const int* pad, const int* stride, float* out)
{
    for (int n = 0; n < N; n++)
        for (int oy = 0; oy < OH; oy++)
            for (int ox = 0; ox < OW; ox++)
                for (int c = 0; c < C; c++)
                {
                    float acc = 0;
                    int count = 0;
                    for (int ky = 0; ky < kernel[0]; ky++)
                        for (int kx = 0; kx < kernel[1]; kx++)
                        {
                            int y = oy * stride[0] - pad[0] + ky;
                            int x = ox * stride[1] - pad[2] + kx;
                            if (0 <= y && y < IH && 0 <= x && x < IW)
                            {
                                acc += in[(((int64_t)n * IH + y) * IW + x) * C + c];
                                count++;
                            }
                        }
                    out[(((int64_t)n * OH + oy) * OW + ox) * C + c] = acc / (float)count;
                }
}

ORC_API int orc_num_procs(void)
{
#ifdef _OPENMP
    return omp_get_num_procs();
#else
    return 1;
#endif
}
