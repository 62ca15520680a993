"""A few CUDA runtime calls through ctypes, for tests that need device memory this library did not allocate."""
import ctypes as C
import glob
import os


def _find():
    roots = [os.environ.get("CUDA_HOME", "/usr/local/cuda")]
    names = []
    for root in roots:
        names += sorted(glob.glob(os.path.join(root, "lib64", "libcudart.so*")), reverse=True)
    try:
        import torch
        names += sorted(glob.glob(os.path.join(os.path.dirname(torch.__file__), "lib", "libcudart*.so*")))
        names += sorted(glob.glob(os.path.join(os.path.dirname(os.path.dirname(torch.__file__)), "nvidia", "cuda_runtime", "lib", "libcudart.so*")))
    except Exception:
        pass
    for name in names:
        try:
            return C.CDLL(name)
        except OSError:
            continue
    raise OSError("libcudart not found")


class Cudart:
    def __init__(self):
        self.rt = _find()
        self.rt.cudaMalloc.argtypes = [C.POINTER(C.c_void_p), C.c_size_t]
        self.rt.cudaMemcpy.argtypes = [C.c_void_p, C.c_void_p, C.c_size_t, C.c_int]
        self.rt.cudaFree.argtypes = [C.c_void_p]

    def _ok(self, rc, what):
        if rc != 0:
            raise RuntimeError(f"{what} failed with CUDA error {rc}")

    def set_device(self, ordinal):
        self._ok(self.rt.cudaSetDevice(ordinal), "cudaSetDevice")

    def malloc(self, nbytes):
        p = C.c_void_p()
        self._ok(self.rt.cudaMalloc(C.byref(p), nbytes), "cudaMalloc")
        return p.value

    def free(self, ptr):
        self._ok(self.rt.cudaFree(ptr), "cudaFree")

    def h2d(self, ptr, array):
        self._ok(self.rt.cudaMemcpy(ptr, array.ctypes.data, array.nbytes, 1), "cudaMemcpy h2d")

    def d2h(self, array, ptr):
        self._ok(self.rt.cudaMemcpy(array.ctypes.data, ptr, array.nbytes, 2), "cudaMemcpy d2h")

    def sync(self):
        self._ok(self.rt.cudaDeviceSynchronize(), "cudaDeviceSynchronize")
