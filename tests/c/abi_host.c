/* Plain C client of the C ABI (no CUDA, no Python): allocator + step builder + argument validation.
 * Built and run by tests/test_capi.py against muxserve_b200/libmuxb200.so. */
#include <stdio.h>
#include <string.h>

#include "muxb200.h"

#define CHECK(c) do { if (!(c)) { printf("FAILED line %d: %s\n", __LINE__, #c); return 1; } } while (0)

int main(void) {
  CHECK(mux_abi_version() >= 1);
  CHECK(strcmp(mux_strerror(MUX_OK), "ok") == 0);

  /* KVStorage(16), L=1, H=2: the known-answer trace of the reference allocator */
  mux_kv_storage_t* kv = mux_kv_storage_create(16);
  CHECK(kv != NULL);
  int32_t rows[] = {1, 2, 0, 2, 2, 0, 3, 2, 0};
  int32_t out[64];
  int64_t n = 0;
  CHECK(mux_kv_storage_allocate_batch(kv, rows, 3, 1, 2, out, 64, &n) == MUX_OK);
  CHECK(n == 13 && out[0] == 3 && out[1] == 4 && out[12] == 15);
  CHECK(mux_kv_storage_new_blocks_allocated(kv) == 12);
  int32_t rows2[] = {1, 1, 1, 2, 1, 1, 3, 1, 1};
  CHECK(mux_kv_storage_allocate_batch(kv, rows2, 3, 1, 2, out, 64, &n) == MUX_OK);
  CHECK(n == 5 && out[0] == 2 && out[1] == 12 && out[4] == 15);      /* request 3 preempted */
  int32_t ids[] = {1, 99};
  CHECK(mux_kv_storage_free_batch(kv, ids, 2) == 6);
  CHECK(mux_kv_storage_check(kv) == MUX_OK);
  mux_kv_storage_destroy(kv);

  /* step builder: logical bookkeeping of one request */
  mux_batch_scheduler_t* bs = mux_batch_scheduler_create(2, 3, 64, 4);
  CHECK(bs != NULL);
  int32_t prompt[6] = {0, 1, 2, 3, 4, 5};
  CHECK(mux_batch_scheduler_add_request(bs, prompt, 6, 11, 5) == MUX_OK);
  int32_t req = 11, info[4];
  CHECK(mux_batch_scheduler_try_batch(bs, &req, 1, NULL, 0, info) == MUX_OK);
  CHECK(info[0] == 11 && info[1] == 2 && info[2] == 0 && info[3] == 2);
  int32_t unknown = 77;
  CHECK(mux_batch_scheduler_try_batch(bs, &unknown, 1, NULL, 0, info) == MUX_ERR_UNKNOWN_REQUEST);
  mux_batch_scheduler_destroy(bs);

  /* device entry points refuse bad arguments before touching a GPU */
  mux_attn_args_t a;
  memset(&a, 0, sizeof a);
  a.dtype = MUX_DTYPE_F16; a.head_size = 64; a.block_size = 16;
  CHECK(mux_paged_attention(&a, NULL, 0, NULL) == MUX_ERR_BAD_HEAD_SIZE);
  CHECK(mux_reshape_and_cache(NULL, NULL) == MUX_ERR_NULL_POINTER);
  printf("c abi ok\n");
  return 0;
}
