/* A plain C99 host of the library: includes the public header, links the shared library and calls
 * the entry points that need no GPU (status, model info, the host-side KV pool). Compiled and run
 * by tests/test_abi_and_host.py; shows that the boundary is a C ABI with no C++ or torch types. */
#include "granite4_b200.h"
#include <stdio.h>
int main(void) {
  granite4_model_info info;
  granite4_status_info st;
  granite4_kv_pool* pool;
  int seq, table[8], ok;
  unsigned int tokens[8] = {1, 2, 3, 4, 5, 6, 7, 8};
  granite4_get_model_info(&info);
  granite4_status(&st);
  printf("%s %s layers=%ld status=%d\n", info.model_id, info.gpu_target, info.num_layers, (int)st.status);
  pool = granite4_kv_pool_create(4, 4);
  seq = granite4_kv_pool_create_sequence(pool);
  ok = granite4_kv_pool_reserve(pool, seq, 8, tokens, 8) && granite4_kv_pool_row_table(pool, seq, 8, table);
  printf("pool ok=%d rows %d %d %d %d | %d\n", ok, table[0], table[1], table[4], table[7],
         (int)granite4_kv_pool_count(pool, GRANITE4_KV_POOL_FREE_PAGES));
  granite4_kv_pool_destroy(pool);
  return ok ? 0 : 1;
}
