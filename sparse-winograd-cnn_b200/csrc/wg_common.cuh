// Shared device helpers for the Winograd F(2x2,3x3) kernels: the three small transforms in
// separable form, plus launch bookkeeping.  Position index t = 4*i + j everywhere.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/winograd2x2_b200.h"

namespace wg {

constexpr int kNumSMs = 148;  // B200: grids of grid-stride kernels are sized in multiples of this

__host__ __device__ inline int cdiv(int a, int b) { return (a + b - 1) / b; }
__host__ __device__ inline long long cdivll(long long a, long long b) { return (a + b - 1) / b; }

__device__ __forceinline__ float4 operator+(float4 a, float4 b) { return make_float4(a.x + b.x, a.y + b.y, a.z + b.z, a.w + b.w); }
__device__ __forceinline__ float4 operator-(float4 a, float4 b) { return make_float4(a.x - b.x, a.y - b.y, a.z - b.z, a.w - b.w); }

// ---- B^T d B, separable: 16 adds for the rows, 16 for the columns -----------------------
// B^T = [[1,0,-1,0],[0,1,1,0],[0,-1,1,0],[0,1,0,-1]]
template <typename T>
__device__ __forceinline__ void bt_d_b(const T (&d)[4][4], T (&v)[4][4])
{
    T r[4][4];
#pragma unroll
    for (int x = 0; x < 4; ++x) {
        r[0][x] = d[0][x] - d[2][x];
        r[1][x] = d[1][x] + d[2][x];
        r[2][x] = d[2][x] - d[1][x];
        r[3][x] = d[1][x] - d[3][x];
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        v[i][0] = r[i][0] - r[i][2];
        v[i][1] = r[i][1] + r[i][2];
        v[i][2] = r[i][2] - r[i][1];
        v[i][3] = r[i][1] - r[i][3];
    }
}

// ---- A^T m A -----------------------------------------------------------------------------
// A^T = [[1,1,1,0],[0,1,-1,-1]]; column step: z[e] from one row of m
__device__ __forceinline__ void at_cols(float m0, float m1, float m2, float m3, float &z0, float &z1)
{
    z0 = m0 + m1 + m2;
    z1 = m1 - m2 - m3;
}
// row step: given the column-transformed pair of Winograd row i, add into y[a][e]
__device__ __forceinline__ void at_rows_accum(int i, float z0, float z1, float (&y)[2][2])
{
    // AT[0] = [1,1,1,0], AT[1] = [0,1,-1,-1]
    if (i == 0) { y[0][0] += z0; y[0][1] += z1; }
    if (i == 1) { y[0][0] += z0; y[0][1] += z1; y[1][0] += z0; y[1][1] += z1; }
    if (i == 2) { y[0][0] += z0; y[0][1] += z1; y[1][0] -= z0; y[1][1] -= z1; }
    if (i == 3) { y[1][0] -= z0; y[1][1] -= z1; }
}

// ---- A dY A^T : the 16 Winograd-domain gradients of a 2x2 output block ---------------------
// dM[i][j] = sum_{a,e} AT[a][i] AT[e][j] g[a][e]
__device__ __forceinline__ void a_g_at(float g00, float g01, float g10, float g11, float (&dm)[4][4])
{
    // rows over a: u[i][e]
    float u[4][2];
    u[0][0] = g00;        u[0][1] = g01;
    u[1][0] = g00 + g10;  u[1][1] = g01 + g11;
    u[2][0] = g00 - g10;  u[2][1] = g01 - g11;
    u[3][0] = -g10;       u[3][1] = -g11;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        dm[i][0] = u[i][0];
        dm[i][1] = u[i][0] + u[i][1];
        dm[i][2] = u[i][0] - u[i][1];
        dm[i][3] = -u[i][1];
    }
}
// one Winograd row i of the above (j = 0..3), used by kernels that walk the rows in turn
__device__ __forceinline__ void a_g_at_row(int i, float g00, float g01, float g10, float g11, float (&dm)[4])
{
    float u0, u1;
    if (i == 0)      { u0 = g00;        u1 = g01; }
    else if (i == 1) { u0 = g00 + g10;  u1 = g01 + g11; }
    else if (i == 2) { u0 = g00 - g10;  u1 = g01 - g11; }
    else             { u0 = -g10;       u1 = -g11; }
    dm[0] = u0; dm[1] = u0 + u1; dm[2] = u0 - u1; dm[3] = -u1;
}

// B^T as compile-time coefficients (for the gather in the input-transform gradient)
__host__ __device__ constexpr int bt_coef(int i, int y)
{
    return (i == 0) ? (y == 0 ? 1 : (y == 2 ? -1 : 0))
         : (i == 1) ? ((y == 1 || y == 2) ? 1 : 0)
         : (i == 2) ? (y == 1 ? -1 : (y == 2 ? 1 : 0))
                    : (y == 1 ? 1 : (y == 3 ? -1 : 0));
}

inline int launch_status()
{
    return cudaGetLastError() == cudaSuccess ? WG2X2_OK : WG2X2_ERR_LAUNCH;
}

}  // namespace wg
