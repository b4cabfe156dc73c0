"""ctypes binding of libbr_host.so (include/br_host.h): the C++ host side -- runtime contexts,
tensor facade and the words machine -- driven from Python for tests and benchmarks."""
import ctypes as C
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "lib", "libbr_host.so")

p, i64, i32, f32, sz, cstr = C.c_void_p, C.c_int64, C.c_int, C.c_float, C.c_size_t, C.c_char_p
SIGNATURES = {
    "brh_last_error": (cstr, []),
    "brh_context_boot": (i32, [i32, p, sz]),
    "brh_context_shutdown": (i32, []),
    "brh_context_stream": (p, []),
    "brh_collective_boot_local": (i32, [i32, i32]),
    "brh_collective_unique_id": (i32, [C.c_char * 128]),
    "brh_collective_boot": (i32, [i32, i32, C.c_char * 128]),
    "brh_collective_split": (i32, [i32]),
    "brh_collective_shutdown": (i32, []),
    "brh_memory_boot": (i32, [sz, i32]),
    "brh_memory_shutdown": (i32, []),
    "brh_env_new": (p, [i32]),
    "brh_env_free": (None, [p]),
    "brh_env_execute": (i32, [p, cstr]),
    "brh_env_build": (p, [p, cstr]),
    "brh_env_run": (i32, [p, p]),
    "brh_program_free": (None, [p]),
    "brh_env_change": (i32, [p, i32]),
    "brh_env_current": (i32, [p]),
    "brh_env_stack_size": (i32, [p]),
    "brh_env_stack_clear": (i32, [p]),
    "brh_env_pop_number": (i32, [p, C.POINTER(C.c_double)]),
    "brh_env_pop_string": (i32, [p, C.c_char_p, sz]),
    "brh_env_push_number": (i32, [p, C.c_double]),
    "brh_env_push_string": (i32, [p, cstr]),
    "brh_env_has": (i32, [p, cstr]),
    "brh_env_get_number": (i32, [p, cstr, C.POINTER(C.c_double)]),
    "brh_env_tensor_info": (i32, [p, cstr, C.POINTER(p), C.POINTER(i32), C.POINTER(i32), C.POINTER(i32), C.POINTER(i64)]),
    "brh_env_tensor_write": (i32, [p, cstr, p, sz]),
    "brh_env_tensor_read": (i32, [p, cstr, p, sz]),
    "brh_env_tensor_write_async": (i32, [p, cstr, p, sz]),
    "brh_last_loss": (f32, []),
    "brh_profile_start": (i32, []),
    "brh_profile_stop": (i32, [C.c_char_p, sz]),
}

_lib = None
_NP = {0: np.float32, 2: np.float16, 3: np.int32}


class HostError(RuntimeError):
    pass


def _preload_bundled_nccl():
    """One NCCL per process: libbr_host.so asks for the soname libnccl.so.2, and a torch imported later needs the
    (newer) build bundled with it under that same soname.  Loading the bundled library first lets both use it;
    without the bundle the system library is used."""
    try:
        import importlib.util
        spec = importlib.util.find_spec("nvidia.nccl")
        if spec and spec.submodule_search_locations:
            for d in spec.submodule_search_locations:
                cand = os.path.join(d, "lib", "libnccl.so.2")
                if os.path.exists(cand):
                    C.CDLL(cand, mode=C.RTLD_GLOBAL)
                    return
    except (ImportError, OSError, ValueError):
        pass


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(f"{LIB_PATH} is missing: run __graft_entry__.build()")
        _preload_bundled_nccl()
        # libbr_host.so finds libbrk.so through its $ORIGIN rpath
        _lib = C.CDLL(LIB_PATH, mode=C.RTLD_GLOBAL)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(_lib, name)
            fn.restype = res
            fn.argtypes = args
    return _lib


def _check(rc):
    if rc != 0:
        raise HostError(lib().brh_last_error().decode(errors="replace"))


def context_boot(device=0, stream=None, workspace_bytes=256 << 20):
    _check(lib().brh_context_boot(device, stream, workspace_bytes))


def context_shutdown():
    _check(lib().brh_context_shutdown())


def collective_boot_local(rank, world):
    _check(lib().brh_collective_boot_local(rank, world))


def collective_unique_id():
    buf = (C.c_char * 128)()
    _check(lib().brh_collective_unique_id(buf))
    return bytes(buf.raw)


def collective_boot(rank, world, id_bytes):
    buf = (C.c_char * 128)(*id_bytes)
    _check(lib().brh_collective_boot(rank, world, buf))


def collective_split(replicas):
    """Splits the booted job into data-parallel replicas of a pipeline (every rank calls it with the same value)."""
    _check(lib().brh_collective_split(int(replicas)))


def collective_shutdown():
    _check(lib().brh_collective_shutdown())


class Env:
    """One words machine (br::Enviroment) with the op.* / io.* words registered."""

    def __init__(self, hash_num=1):
        self._h = lib().brh_env_new(hash_num)
        if not self._h:
            raise HostError(lib().brh_last_error().decode())

    def close(self):
        if self._h:
            lib().brh_env_free(self._h)
            self._h = None

    def __del__(self):
        self.close()

    def execute(self, text):
        _check(lib().brh_env_execute(self._h, text.encode()))

    def build(self, text):
        """Compile + link; returns a program handle for run() (free it with free_program)."""
        h = lib().brh_env_build(self._h, text.encode())
        if not h:
            raise HostError(lib().brh_last_error().decode(errors="replace"))
        return h

    def run(self, program):
        _check(lib().brh_env_run(self._h, program))

    @staticmethod
    def free_program(program):
        lib().brh_program_free(program)

    def change(self, index):
        _check(lib().brh_env_change(self._h, index))

    @property
    def current(self):
        return lib().brh_env_current(self._h)

    @property
    def stack_size(self):
        return lib().brh_env_stack_size(self._h)

    def clear_stack(self):
        _check(lib().brh_env_stack_clear(self._h))

    def pop_number(self):
        v = C.c_double()
        _check(lib().brh_env_pop_number(self._h, C.byref(v)))
        return v.value

    def pop_string(self):
        buf = C.create_string_buffer(4096)
        _check(lib().brh_env_pop_string(self._h, buf, 4096))
        return buf.value.decode()

    def push_number(self, v):
        _check(lib().brh_env_push_number(self._h, float(v)))

    def push_string(self, s):
        _check(lib().brh_env_push_string(self._h, s.encode()))

    def has(self, name):
        return bool(lib().brh_env_has(self._h, name.encode()))

    def get_number(self, name):
        v = C.c_double()
        _check(lib().brh_env_get_number(self._h, name.encode(), C.byref(v)))
        return v.value

    def tensor_info(self, name):
        data, cuda, dt, nd = p(), i32(), i32(), i32()
        dims = (i64 * 8)()
        _check(lib().brh_env_tensor_info(self._h, name.encode(), C.byref(data), C.byref(cuda), C.byref(dt), C.byref(nd), dims))
        return {"data": data.value, "cuda": bool(cuda.value), "dtype": dt.value, "shape": tuple(dims[i] for i in range(nd.value))}

    def write(self, name, array):
        info = self.tensor_info(name)
        a = np.ascontiguousarray(array, dtype=_NP[info["dtype"]])
        assert a.size == int(np.prod(info["shape"])), (name, a.shape, info["shape"])
        _check(lib().brh_env_tensor_write(self._h, name.encode(), a.ctypes.data_as(p), a.nbytes))

    def write_async(self, name, array):
        """Queues the write on the compute stream (the data is copied out of `array` before this returns)."""
        info = self.tensor_info(name)
        a = np.ascontiguousarray(array, dtype=_NP[info["dtype"]])
        assert a.size == int(np.prod(info["shape"])), (name, a.shape, info["shape"])
        _check(lib().brh_env_tensor_write_async(self._h, name.encode(), a.ctypes.data_as(p), a.nbytes))

    def read(self, name):
        info = self.tensor_info(name)
        a = np.empty(info["shape"], dtype=_NP[info["dtype"]])
        _check(lib().brh_env_tensor_read(self._h, name.encode(), a.ctypes.data_as(p), a.nbytes))
        return a


def profile_start():
    _check(lib().brh_profile_start())


def profile_stop():
    """Returns {family: {"ms": device milliseconds, "calls": launches}} and switches profiling off."""
    import json
    buf = C.create_string_buffer(1 << 16)
    _check(lib().brh_profile_stop(buf, 1 << 16))
    return json.loads(buf.value.decode())


def last_loss():
    return float(lib().brh_last_loss())
