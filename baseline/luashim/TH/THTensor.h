/* Stand-in for Torch7's TH: a float tensor is a data pointer and an element count. */
#ifndef SHIM_THTENSOR_H
#define SHIM_THTENSOR_H
typedef struct THFloatTensor {
  float* data;
  long n;
} THFloatTensor;

static inline long THFloatTensor_nElement(const THFloatTensor* t) { return t->n; }
static inline float* THFloatTensor_data(const THFloatTensor* t) { return t->data; }
void THError(const char* fmt, ...);
#endif
