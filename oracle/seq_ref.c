/* Plain-C restatement of the order-sensitive index algorithms -- TEST
 * INFRASTRUCTURE ONLY (never linked into the product).
 *
 * The reference hands these operators to its vendor library
 * (topsatenScatterAdd / topsatenIndexPutImpl / topsatenIndexSelect /
 * topsatenGather / topsatenCopy; call sites: generated aotops::scatter_add_out,
 * torch_gcu/csrc/aten/aot_ops/gcu_tensor_advanced_indexing.cpp:60-90,
 * generated aotops::index_select / gather_out,
 * torch_gcu/csrc/aten/aot_ops/gcu_copy.cpp:108-130) and defines their result as
 * the CPU ATen result. These loops restate that result independently of ATen:
 * each destination receives its addends one by one in ascending source order,
 * in the element type. The tests check ATen against these loops, which pins
 * the accumulation order the CUDA kernels must reproduce.
 */
#include <stdint.h>
#include <string.h>

/* out (n_dst, inner) starts as self; out[rows[i]] += src[i] for i ascending. */
void seq_scatter_add_rows_f32(float* out, const float* self, const int64_t* rows,
                              const float* src, int64_t n_src, int64_t n_dst, int64_t inner) {
  if (out != self) memcpy(out, self, (size_t)(n_dst * inner) * sizeof(float));
  for (int64_t i = 0; i < n_src; ++i) {
    int64_t r = rows[i];
    if (r < 0) r += n_dst;
    if (r < 0 || r >= n_dst) continue;
    volatile float* o = out + r * inner;
    const float* s = src + i * inner;
    for (int64_t j = 0; j < inner; ++j) o[j] = o[j] + s[j];
  }
}

/* generic 2-D scatter_add along dim 0 with a full-shape index */
void seq_scatter_add_dim0_f32(float* out, const float* self, const int64_t* index,
                              const float* src, int64_t n_src, int64_t n_dst, int64_t inner) {
  if (out != self) memcpy(out, self, (size_t)(n_dst * inner) * sizeof(float));
  for (int64_t i = 0; i < n_src; ++i)
    for (int64_t j = 0; j < inner; ++j) {
      int64_t r = index[i * inner + j];
      if (r < 0 || r >= n_dst) continue;
      volatile float* o = out + r * inner + j;
      *o = *o + src[i * inner + j];
    }
}

/* index_put without accumulate: last writer (highest i) wins */
void seq_index_put_rows_f32(float* out, const int64_t* rows, const float* src, int64_t n_src,
                            int64_t n_dst, int64_t inner) {
  for (int64_t i = 0; i < n_src; ++i) {
    int64_t r = rows[i];
    if (r < 0) r += n_dst;
    if (r < 0 || r >= n_dst) continue;
    memcpy(out + r * inner, src + i * inner, (size_t)inner * sizeof(float));
  }
}

/* row gather of `row_bytes`-byte rows: index_select(dim 0) / embedding */
void seq_gather_rows(uint8_t* out, const uint8_t* table, const int64_t* rows, int64_t n,
                     int64_t row_bytes) {
  for (int64_t i = 0; i < n; ++i) memcpy(out + i * row_bytes, table + rows[i] * row_bytes, (size_t)row_bytes);
}

/* gather along the last dim of a (rows, cols_self) fp32 matrix */
void seq_gather_lastdim_f32(float* out, const float* self, const int64_t* index, int64_t rows,
                            int64_t cols_index, int64_t cols_self) {
  for (int64_t i = 0; i < rows; ++i)
    for (int64_t j = 0; j < cols_index; ++j)
      out[i * cols_index + j] = self[i * cols_self + index[i * cols_index + j]];
}

/* fp32 -> bf16 bits: round to nearest even, NaN -> 0x7FC0 (c10::BFloat16) */
void seq_f32_to_bf16(uint16_t* out, const float* in, int64_t n) {
  for (int64_t i = 0; i < n; ++i) {
    uint32_t u;
    memcpy(&u, in + i, 4);
    if ((u & 0x7fffffffu) > 0x7f800000u) { out[i] = 0x7FC0; continue; }
    u += 0x7FFFu + ((u >> 16) & 1u);
    out[i] = (uint16_t)(u >> 16);
  }
}

void seq_bf16_to_f32(float* out, const uint16_t* in, int64_t n) {
  for (int64_t i = 0; i < n; ++i) {
    uint32_t u = (uint32_t)in[i] << 16;
    memcpy(out + i, &u, 4);
  }
}
