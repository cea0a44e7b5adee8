// nextDoorPythonModule.cu -- Python module glue with the functions of the reference's
// src/nextDoorPythonModule.cu:40-132: initSampling(graph), sample(), finalSamples(),
// finalSampleLength(), freeDeviceMemory(), and the C symbol finalSamplesArray() for ctypes.
// Use exactly as there: include this file at the end of the application file after defining
// INIT_FUNC_NAME, `const char* moduleName` and a static `nextDoorData` object, with -DPYTHON_3.
#include <Python.h>

#include "nextdoor.cu"

static CSR *graph_csr = nullptr;
static Graph graph;

static PyObject *initSampling(PyObject *, PyObject *args) {
  char *graph_file;
  if (!PyArg_ParseTuple(args, "s", &graph_file)) return NULL;
  graph_csr = loadGraph(graph, graph_file, (char *)"edge-list", (char *)"binary");
  if (graph_csr == nullptr) { PyErr_SetString(PyExc_RuntimeError, nd_last_error()); return NULL; }
  if (!allocNextDoorDataOnGPU(graph_csr, nextDoorData)) { PyErr_SetString(PyExc_RuntimeError, "allocNextDoorDataOnGPU failed"); return NULL; }
  nextDoorData.gpuCSRPartitions = transferCSRToGPUs(nextDoorData, graph_csr);
  Py_RETURN_NONE;
}

static PyObject *sample(PyObject *, PyObject *) {  // the sample-parallel path, as in the reference (:54-58)
  if (!doSampleParallelSampling(graph_csr, nextDoorData)) { PyErr_SetString(PyExc_RuntimeError, nd_last_error()); return NULL; }
  Py_RETURN_NONE;
}

static PyObject *finalSamples(PyObject *, PyObject *) {
  std::vector<VertexID_t> &fin = getFinalSamples(nextDoorData);
  PyObject *result = PyList_New((Py_ssize_t)fin.size());
  for (size_t i = 0; i < fin.size(); i++) PyList_SET_ITEM(result, (Py_ssize_t)i, PyLong_FromLong(fin[i]));
  return result;
}

static PyObject *finalSampleLength(PyObject *, PyObject *) {
  return Py_BuildValue("n", (Py_ssize_t)nextDoorData.hFinalSamples.size());
}

static PyObject *freeDeviceMemory(PyObject *, PyObject *) {
  freeDeviceData(nextDoorData);
  Py_RETURN_NONE;
}

extern "C" int *finalSamplesArray() { return &getFinalSamples(nextDoorData)[0]; }

static PyMethodDef ModuleMethods[] = {
    {"initSampling", initSampling, METH_VARARGS, "initSampling(graph): load a binary edge-list graph and allocate the samples."},
    {"sample", sample, METH_VARARGS, "sample(): run the sampling on the GPU."},
    {"finalSamples", finalSamples, METH_VARARGS, "finalSamples(): the final samples as a Python list."},
    {"finalSampleLength", finalSampleLength, METH_VARARGS, "finalSampleLength(): number of vertex slots in the final samples."},
    {"freeDeviceMemory", freeDeviceMemory, METH_VARARGS, "freeDeviceMemory(): release the device memory."},
    {NULL, NULL, 0, NULL}};

static struct PyModuleDef SamplingModule = {PyModuleDef_HEAD_INIT, moduleName, NULL, -1, ModuleMethods};
extern "C" PyMODINIT_FUNC INIT_FUNC_NAME(void) { return PyModule_Create(&SamplingModule); }
