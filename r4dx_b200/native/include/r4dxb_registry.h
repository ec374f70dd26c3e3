/* Machine-readable registry of the kernels behind r4dxb.h (host library; no device needed to query it). */
#ifndef R4DXB_REGISTRY_H_
#define R4DXB_REGISTRY_H_

#ifdef __cplusplus
extern "C" {
#endif

enum {
  R4DXB_C_EQ = 0,  /* param == ival */
  R4DXB_C_LE = 1,  /* param <= ival */
  R4DXB_C_GE = 2,  /* param >= ival */
  R4DXB_C_DIV = 3, /* param % ival == 0 */
  R4DXB_C_IN = 4,  /* param is one of the space-separated decimal words of sval */
};

typedef struct R4dxbConstraint {
  const char* key; /* parameter name: T (rows), N, K, kb, D (head dim), world, ... */
  int op;
  long long ival;
  const char* sval;
} R4dxbConstraint;

typedef struct R4dxbKernelInfo {
  const char* name;     /* entry point without the r4dxb_ prefix */
  const char* family;   /* gemm | gemm+collective | collective | attn | gdn | moe | quant | sampling | elementwise | conv | dflash */
  const char* op;       /* the operation callers select on; several kernels may share one */
  const char* computes; /* for a human */
  const char* shape;    /* geometry, for a human */
  const char* dtypes;
  const char* engine;   /* tcgen05 | mma.sync | simt, "+bulk-copy" / "+peer-stores" where they apply */
  const R4dxbConstraint* constraints;
  int n_constraints;
} R4dxbKernelInfo;

int r4dxb_kernel_count(void);
const R4dxbKernelInfo* r4dxb_kernel_at(int i);
int r4dxb_kernel_covers(const char* name, const char* const* keys, const long long* vals, int n);

#ifdef __cplusplus
}
#endif
#endif
