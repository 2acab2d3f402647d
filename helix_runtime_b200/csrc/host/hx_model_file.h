/* Helix's native model file ("HELIXLM1"): a checked, memory-mapped reader.  Host code only.
 *
 * hx_model_file_open maps the file and checks the header and the tensor directory against the
 * layout that the model's sizes imply; hx_model_file_verify then checks the alignment padding
 * (zero bytes), every payload's FNV-1a checksum and that every value is finite.  Tensors are
 * read in place: hx_model_tensor.data points into the mapping, which lives until
 * hx_model_file_close.  Every function returns 0 or a negative code and leaves a message for
 * hx_host_last_error() (per thread).
 *
 * Tensors are the reference's: float32, [in, out] for the projections, the rows of the query
 * and key projections ordered for adjacent-pair rotation (tools/convert_hf_llama.py:400-542).
 */
#ifndef HELIX_B200_MODEL_FILE_H
#define HELIX_B200_MODEL_FILE_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define HX_FILE_OK 0
#define HX_FILE_IO (-1)        /* the file could not be opened, inspected or mapped */
#define HX_FILE_FORMAT (-2)    /* the file is not a well-formed model file */
#define HX_FILE_ARGUMENT (-3)

#define HX_MODEL_KIND_LLAMA 1

enum hx_tensor_role {
  HX_ROLE_TOKEN_EMBEDDING = 1, HX_ROLE_ATTENTION_NORM = 2, HX_ROLE_QUERY = 3, HX_ROLE_KEY = 4,
  HX_ROLE_VALUE = 5, HX_ROLE_ATTENTION_OUTPUT = 6, HX_ROLE_FFN_NORM = 7, HX_ROLE_GATE = 8,
  HX_ROLE_UP = 9, HX_ROLE_DOWN = 10, HX_ROLE_FINAL_NORM = 11, HX_ROLE_LM_HEAD = 12
};

typedef struct hx_model_config {
  uint64_t vocab_size, hidden_size, intermediate_size, num_layers, num_heads, max_positions;
  float rms_norm_eps, rope_theta;
  uint32_t model_kind;
} hx_model_config;

typedef struct hx_model_tensor {
  int role;            /* hx_tensor_role */
  int layer;           /* -1 for the embedding, the final norm and the head */
  int rank;
  uint64_t dims[4];
  uint64_t offset, bytes, checksum;
  const void* data;    /* float32 little-endian, inside the mapping */
} hx_model_tensor;

typedef struct hx_model_file hx_model_file;

const char* hx_host_last_error(void);
/* FNV-1a over `count` bytes, continuing from `seed` (0: the standard offset basis) */
uint64_t hx_fnv1a64(const void* bytes, uint64_t count, uint64_t seed);

int hx_model_file_open(const char* path, hx_model_file** out);
void hx_model_file_close(hx_model_file* file);
int hx_model_file_config(const hx_model_file* file, hx_model_config* out);
long long hx_model_file_tensor_count(const hx_model_file* file);
int hx_model_file_tensor(const hx_model_file* file, long long index, hx_model_tensor* out);
int hx_model_file_verify(const hx_model_file* file, int threads);

#ifdef __cplusplus
}
#endif
#endif
