/* Golden driver: links against the reference's own sources (g2b.h API), feeds the
 * given token ids one by one through model_forward and writes the f32 logits of
 * every position to a file.  Built and run only by make_golden.py. */
#include "g2b.h"
#include <stdlib.h>
#include <string.h>

int main(int argc, char **argv) {
  if (argc < 4) { fprintf(stderr, "usage: dump_logits model.g2bx out.bin id,id,...\n"); return 1; }
  Model m;
  if (model_load_g2bx(argv[1], &m)) return 1;
  FILE *out = fopen(argv[2], "wb");
  if (!out) return 1;
  f32 *logits = malloc((size_t)m.c.vocab * sizeof(f32));
  int pos = 0;
  for (char *t = strtok(argv[3], ","); t; t = strtok(NULL, ",")) {
    model_forward(&m, atoi(t), pos++, logits);
    fwrite(logits, sizeof(f32), (size_t)m.c.vocab, out);
  }
  fclose(out);
  free(logits);
  model_free(&m);
  return 0;
}
