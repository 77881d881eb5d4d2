/* A model library that touches no GPU: it only exercises the calling protocol, so the loader
 * can be tested on a CPU-only machine.  init hoists three "tensors" whose descriptors are
 * malloc'ed int64 arrays holding a tag; forward(x: memref, k: int32) returns a malloc'ed record
 * of everything it received, in order. */
#include <stdint.h>
#include <stdlib.h>

typedef struct {
  int64_t rank;
  void *descriptor;
} Unranked;

static int init_calls = 0;

void _hom_ciface_forward_argNum(void **args) { *(int32_t *)args[0] = 3; }

void _hom_ciface_forward_initFn(void **args) {
  Unranked *out = (Unranked *)args[0];
  ++init_calls;
  for (int i = 0; i < 3; ++i) {
    int64_t *d = (int64_t *)malloc(sizeof(int64_t) * 4);
    d[0] = 1000 + i;
    out[i].rank = i + 1;
    out[i].descriptor = d;
  }
}

void _hom_ciface_forward(void **args) {
  int64_t *rec = (int64_t *)malloc(sizeof(int64_t) * 12);
  for (int i = 0; i < 3; ++i) {
    rec[2 * i] = *(int64_t *)args[2 * i];                   /* rank of hoisted tensor i */
    rec[2 * i + 1] = **(int64_t **)args[2 * i + 1];         /* its tag */
  }
  rec[6] = *(int64_t *)args[6];                             /* user memref: rank */
  rec[7] = **(int64_t **)args[7];                           /* first word of its descriptor */
  rec[8] = *(int32_t *)args[8];                             /* user int32 */
  rec[9] = init_calls;
  Unranked r = {2, rec};
  *(Unranked *)args[9] = r;
}
