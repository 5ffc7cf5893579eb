/*
 * _dxb_fast: a compiled binding for the one call that sits on the eager hot path.
 *
 * ctypes converts each of dxb_wq_gemm_ex's 17 arguments through its own machinery on every
 * call (about 4 us in all); this module parses them with the CPython fast-call convention
 * and calls the same C-ABI entry point of libdexter_b200.so.  It contains no compute and no
 * fallback: ops.py uses it when it has been built and bound, and ctypes otherwise; either
 * way the work is done by dxb_wq_gemm_ex.
 *
 *   bind(handle)      address of dxb_wq_gemm_ex (an int, taken from the loaded library)
 *   gemm(bits, x, ldx, qweight, scales, zeros, bias, out, ldo, M, N, K, group_size,
 *        workspace, workspace_bytes, layout, epilogue, max_ctas, serialize, stream) -> rc
 *
 * Pointers travel as Python ints (0 = NULL).  Calls with a fused sum over ranks keep using
 * ctypes (they carry a pointer table and are not the latency-critical single-GPU path).
 */
#define PY_SSIZE_T_CLEAN
#include <Python.h>
#include <stdint.h>

#include "../../include/dexter_b200.h"

typedef int (*gemm_ex_fn)(int, const void*, int64_t, const void*, const void*, const void*, const void*,
                          void*, int64_t, int, int, int, int, void*, size_t, const dxb_gemm_opts*, void*);
static gemm_ex_fn g_gemm = NULL;

static PyObject* fast_bind(PyObject* self, PyObject* arg) {
  (void)self;
  void* p = PyLong_AsVoidPtr(arg);
  if (p == NULL && PyErr_Occurred()) return NULL;
  g_gemm = (gemm_ex_fn)p;
  Py_RETURN_NONE;
}

static int as_i64(PyObject* o, int64_t* out) {
  const long long v = PyLong_AsLongLong(o);
  if (v == -1 && PyErr_Occurred()) return 0;
  *out = (int64_t)v;
  return 1;
}
static int as_ptr(PyObject* o, void** out) {
  const unsigned long long v = PyLong_AsUnsignedLongLong(o);
  if (v == (unsigned long long)-1 && PyErr_Occurred()) return 0;
  *out = (void*)(uintptr_t)v;
  return 1;
}

static PyObject* fast_gemm(PyObject* self, PyObject* const* a, Py_ssize_t n) {
  (void)self;
  if (g_gemm == NULL) {
    PyErr_SetString(PyExc_RuntimeError, "_dxb_fast.gemm called before bind()");
    return NULL;
  }
  if (n != 20) {
    PyErr_SetString(PyExc_TypeError, "_dxb_fast.gemm takes exactly 20 integer arguments");
    return NULL;
  }
  int64_t v[20];
  void* p[20];
  /* which of the 20 are pointers */
  static const char is_ptr[20] = {0, 1, 0, 1, 1, 1, 1, 1, 0, 0, 0, 0, 0, 1, 0, 0, 0, 0, 0, 1};
  for (int i = 0; i < 20; ++i) {
    if (is_ptr[i]) {
      if (!as_ptr(a[i], &p[i])) return NULL;
    } else if (!as_i64(a[i], &v[i])) {
      return NULL;
    }
  }
  dxb_gemm_opts opts;
  opts.weight_layout = (int)v[15];
  opts.epilogue = (int)v[16];
  opts.max_ctas = (int)v[17];
  opts.peer_world = 0;
  opts.peer_rank = 0;
  opts.peer_regions = NULL;
  opts.peer_capacity_elems = 0;
  opts.serialize = (int)v[18];
  const int rc = g_gemm((int)v[0], p[1], v[2], p[3], p[4], p[5], p[6], p[7], v[8], (int)v[9], (int)v[10],
                        (int)v[11], (int)v[12], p[13], (size_t)v[14], &opts, p[19]);
  return PyLong_FromLong(rc);
}

static PyMethodDef fast_methods[] = {
    {"bind", (PyCFunction)fast_bind, METH_O, "bind(address of dxb_wq_gemm_ex)"},
    {"gemm", (PyCFunction)(void (*)(void))fast_gemm, METH_FASTCALL, "dxb_wq_gemm_ex with plain integers"},
    {NULL, NULL, 0, NULL}};

static struct PyModuleDef fast_module = {PyModuleDef_HEAD_INIT, "_dxb_fast",
                                         "compiled binding of dxb_wq_gemm_ex", -1, fast_methods,
                                         NULL, NULL, NULL, NULL};

PyMODINIT_FUNC PyInit__dxb_fast(void) { return PyModule_Create(&fast_module); }
