/* A CPython extension with ONE job: hand the seven scalars of a fixed-size collective to purlin_call_fixed without the
 * argument conversion of a ctypes foreign call (measured on the host with the launch stubbed out: 1.4 us per call through
 * ctypes, 0.45 us through this module; a small collective costs about 10 us of host time per launch in all).
 *
 * The module links against nothing: Python passes it the address of the library's entry point (bind), so the same file
 * serves whichever library was loaded. The reference gets the same effect from its pybind11 module
 * (purlin/bindings.py:16-453 of the reference).
 */
#define PY_SSIZE_T_CLEAN
#include <Python.h>
#include <stddef.h>

typedef int (*call_fixed_fn)(void*, int, const void*, void*, size_t, unsigned, void*);
static call_fixed_fn g_call_fixed = NULL;

static PyObject* fc_bind(PyObject* self, PyObject* address) {
  (void)self;
  void* p = PyLong_AsVoidPtr(address);
  if (p == NULL && PyErr_Occurred()) return NULL;
  g_call_fixed = (call_fixed_fn)p;
  Py_RETURN_NONE;
}

/* call_fixed(ctx, collective, src, dst, bytes, traits, stream) -> status of purlin_call_fixed */
static PyObject* fc_call_fixed(PyObject* self, PyObject* const* args, Py_ssize_t nargs) {
  (void)self;
  if (nargs != 7) { PyErr_SetString(PyExc_TypeError, "call_fixed takes (ctx, collective, src, dst, bytes, traits, stream)"); return NULL; }
  if (g_call_fixed == NULL) { PyErr_SetString(PyExc_RuntimeError, "call_fixed: no entry point bound"); return NULL; }
  void* ctx = PyLong_AsVoidPtr(args[0]);
  const long collective = PyLong_AsLong(args[1]);
  void* src = PyLong_AsVoidPtr(args[2]);
  void* dst = PyLong_AsVoidPtr(args[3]);
  const size_t bytes = PyLong_AsSize_t(args[4]);
  const unsigned long traits = PyLong_AsUnsignedLong(args[5]);
  void* stream = PyLong_AsVoidPtr(args[6]);
  if (PyErr_Occurred()) return NULL;
  int rc;
  Py_BEGIN_ALLOW_THREADS                      /* a launch can block while the stream's queue is full */
  rc = g_call_fixed(ctx, (int)collective, src, dst, bytes, (unsigned)traits, stream);
  Py_END_ALLOW_THREADS
  return PyLong_FromLong(rc);
}

static PyMethodDef fc_methods[] = {
    {"bind", fc_bind, METH_O, "bind(address of purlin_call_fixed)"},
    {"call_fixed", (PyCFunction)(void (*)(void))fc_call_fixed, METH_FASTCALL, "call_fixed(ctx, collective, src, dst, bytes, traits, stream) -> int"},
    {NULL, NULL, 0, NULL}};

static struct PyModuleDef fc_module = {PyModuleDef_HEAD_INIT, "_purlin_fastcall", "scalar fast path into libpurlin", -1, fc_methods, NULL, NULL, NULL, NULL};

PyMODINIT_FUNC PyInit__purlin_fastcall(void) { return PyModule_Create(&fc_module); }
