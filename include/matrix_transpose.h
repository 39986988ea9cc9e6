/*! \file matrix_transpose.h
 *  \brief odata[n*M + m] = idata[m*N + n]; same signature as the reference's
 *  src/include/matrix_transpose.h:3-4 (definition src/transpose/transpose.cu:60-77), for any 1- or
 *  2-byte element type and any M, N (the reference handles bf16 with M % 64 == 0, N % 32 == 0 only).
 *  Device pointers; default stream; asynchronous. Defined in libqgemm.so for __nv_bfloat16, __half,
 *  int8_t, uint8_t, uint16_t and __nv_fp8_e4m3.
 */
#pragma once

template <typename T>
void matrix_transpose(const T* idata, T* odata, int M, int N);
