/* Compiled by tests/test_host.py with plain gcc: the public header must be valid C (not only C++), and the
 * layout of struct rewb200_config that a C compiler sees is printed field by field so that the ctypes mirror
 * (rew_b200/_lib.py) and the generated Nim object (nim/rew_b200_abi.nim) can be compared with it. */
#include <stddef.h>
#include <stdio.h>

#include "rew_b200.h"

#define FIELD(name) printf("%s %zu %zu\n", #name, offsetof(rewb200_config, name), sizeof(((rewb200_config*)0)->name))

int main(void) {
  FIELD(vocab); FIELD(d_model); FIELD(n_layers); FIELD(n_heads); FIELD(n_kv_heads); FIELD(head_dim); FIELD(ffn);
  FIELD(max_seq); FIELD(theta); FIELD(eps); FIELD(norm_kind); FIELD(mask_kind); FIELD(n_routed); FIELD(n_shared);
  FIELD(top_k); FIELD(moe_ffn); FIELD(first_dense); FIELD(dtype); FIELD(tp_rank); FIELD(tp_size); FIELD(ep_rank);
  FIELD(ep_size); FIELD(weight_quant);
  printf("sizeof %zu %d\n", sizeof(rewb200_config), REWB200_BF16);
  /* every entry point is declared with C linkage: taking an address needs only the declaration */
  int (*init)(const int*, int) = rewb200_init;
  int (*disp)(const char*, rewb200_buffer* const*, int, const char* const*, const char* const*, int, rewb200_buffer**, int*) =
      rewb200_dispatch;
  (void)init;
  (void)disp;
  return 0;
}
