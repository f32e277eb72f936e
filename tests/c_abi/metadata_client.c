/* A plain C99 client of the C ABI (no C++, no Python, no torch): what a cgo / JNI / pybind
 * binding of the reference would link against.  It calls the host-side metadata entry points
 * (random-block table, CSR block table, varlen offsets) and prints what it got, one integer per
 * line; tests/test_c_abi.py compiles it with gcc, links it against libraptor_b200.so and compares
 * the output with the oracle.  Usage: metadata_client <layer_seed> <len_tokens>... */
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "raptor_b200.h"

static void die(const char* what) {
  fprintf(stderr, "%s: %s\n", what, rt_last_error());
  exit(1);
}

int main(int argc, char** argv) {
  if (argc < 3) return 2;
  const unsigned seed = (unsigned)atoi(argv[1]);
  const int n_seq = argc - 2;
  int32_t* lens = (int32_t*)malloc(sizeof(int32_t) * (size_t)n_seq);
  int n_blocks = 0;
  for (int i = 0; i < n_seq; ++i) {
    lens[i] = atoi(argv[2 + i]);
    n_blocks += lens[i] / 64;
  }
  rt_config cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.hidden = 768; cfg.heads = 12; cfg.ffn = 3072; cfg.layers = 12; cfg.block = 64; cfg.num_rand = 3;
  cfg.max_pos = 4096; cfg.vocab = 50358; cfg.type_vocab = 2; cfg.pattern = RT_PATTERN_BIGBIRD;
  cfg.dtype = RT_F16; cfg.eps = 1e-12f;

  printf("version %d\n", rt_version());

  int32_t* prefix = (int32_t*)malloc(sizeof(int32_t) * (size_t)(n_seq + 1));
  if (rt_seq_block_prefix(lens, n_seq, cfg.block, prefix) != RT_OK) die("rt_seq_block_prefix");
  printf("prefix");
  for (int i = 0; i <= n_seq; ++i) printf(" %d", prefix[i]);
  printf("\n");

  int64_t visits = 0;
  if (rt_count_visits(&cfg, lens, n_seq, &visits) != RT_OK) die("rt_count_visits");
  printf("visits %lld\n", (long long)visits);

  int32_t* kv_ptr = (int32_t*)malloc(sizeof(int32_t) * (size_t)(n_blocks + 1));
  int32_t* kv_idx = (int32_t*)malloc(sizeof(int32_t) * (size_t)(visits * cfg.heads));
  if (rt_build_block_csr(&cfg, seed, lens, n_seq, kv_ptr, kv_idx) != RT_OK) die("rt_build_block_csr");
  printf("kv_ptr");
  for (int i = 0; i <= n_blocks; ++i) printf(" %d", kv_ptr[i]);
  printf("\nkv_idx");
  for (long long i = 0; i < (long long)visits * cfg.heads; ++i) printf(" %d", kv_idx[i]);
  printf("\n");

  /* an unsupported length is an error code and a message, not a crash: 768 tokens = 12 blocks,
   * where the validation model's random ids leave the sequence */
  int32_t table[12 * 10 * 3];
  rt_status s = rt_rand_block_table(seed, 12, 12, 3, 4096, 64, table);
  printf("bad_status %d\n", (int)s);
  printf("bad_message_chars %d\n", (int)strlen(rt_last_error()));
  free(lens); free(prefix); free(kv_ptr); free(kv_idx);
  return 0;
}
