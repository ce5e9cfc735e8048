"""ctypes view of include/gradc_trainer.h: the host-side training step (forward, Tensor::backward(), clip, AdamW)."""
import ctypes
import os

import numpy as np

from . import capi

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libgradc_trainer.so")
_LIB = None


def _lib():
    global _LIB
    if _LIB is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError("%s is missing: build it with `python -c 'import __graft_entry__ as g; g.build()'`" % LIB_PATH)
        capi.lib()  # the kernel library first, so both share one copy
        L = ctypes.CDLL(LIB_PATH)
        L.gct_last_error.restype = ctypes.c_char_p
        vp, i64, f32, ci = ctypes.c_void_p, ctypes.c_int64, ctypes.c_float, ctypes.c_int
        L.gct_create.argtypes = [ctypes.c_char_p] + [i64] * 6 + [f32] * 8 + [ci, ctypes.POINTER(vp)]
        L.gct_destroy.argtypes = [vp]
        for n in ("gct_num_tensors", "gct_num_params", "gct_launch_count", "gct_arena_high_water_bytes", "gct_num_buckets"):
            getattr(L, n).argtypes, getattr(L, n).restype = [vp], i64
        L.gct_param_info.argtypes = [vp, i64, ctypes.c_char_p, i64, ctypes.POINTER(i64), ctypes.POINTER(ci)]
        for n in ("gct_set_param", "gct_get_param", "gct_get_grad"):
            getattr(L, n).argtypes = [vp, ctypes.c_char_p, vp, i64]
        L.gct_set_lr.argtypes = [vp, f32]
        L.gct_zero_grad.argtypes = [vp]
        L.gct_forward_backward.argtypes = [vp, vp, vp, ci, i64, i64, i64, ctypes.POINTER(f32)]
        L.gct_optimizer_step.argtypes = [vp, ctypes.POINTER(f32)]
        L.gct_sync.argtypes = [vp]
        L.gct_generate.argtypes = [vp, vp, i64, i64, i64, i64, f32, i64, vp]
        L.gct_save_checkpoint.argtypes = [vp, ctypes.c_char_p, ctypes.c_char_p]
        L.gct_load_checkpoint.argtypes = [vp, ctypes.c_char_p, ctypes.c_char_p]
        L.gct_stream.argtypes, L.gct_stream.restype = [vp], vp
        L.gct_context.argtypes, L.gct_context.restype = [vp], vp
        L.gct_dp_init.argtypes = [vp, vp, ci, ci, i64]
        _LIB = L
    return _LIB


class TrainerError(RuntimeError):
    pass


def _ptr(a):
    if hasattr(a, "data_ptr"):
        return ctypes.c_void_p(a.data_ptr())
    return ctypes.c_void_p(a.ctypes.data)


class Trainer:
    def __init__(self, arch, V, T, C, H, L, F, lr=3e-4, beta1=0.9, beta2=0.95, wd=0.1, eps=1e-5, norm_eps=1e-5, ce_eps=1e-5, clip=0.0, device=0):
        self.L = _lib()
        self.h = ctypes.c_void_p()
        self.shape = dict(arch=arch, V=V, T=T, C=C, H=H, L=L, F=F)
        self._ok(self.L.gct_create(arch.encode(), V, T, C, H, L, F, lr, beta1, beta2, wd, eps, norm_eps, ce_eps, clip, device, ctypes.byref(self.h)))

    def _ok(self, rc):
        if rc != 0:
            raise TrainerError(self.L.gct_last_error().decode())

    def params(self):
        """[(name, n_elements, no_decay)] in arena order."""
        out = []
        buf = ctypes.create_string_buffer(256)
        n, nd = ctypes.c_int64(), ctypes.c_int()
        for i in range(self.L.gct_num_tensors(self.h)):
            self._ok(self.L.gct_param_info(self.h, i, buf, 256, ctypes.byref(n), ctypes.byref(nd)))
            out.append((buf.value.decode(), n.value, bool(nd.value)))
        return out

    def num_params(self):
        return self.L.gct_num_params(self.h)

    def load(self, weights):
        for name, n, _ in self.params():
            a = np.ascontiguousarray(weights[name], dtype=np.float32)
            assert a.size == n, name
            self._ok(self.L.gct_set_param(self.h, name.encode(), _ptr(a), n))

    def get(self, what="param"):
        fn = self.L.gct_get_param if what == "param" else self.L.gct_get_grad
        out = {}
        for name, n, _ in self.params():
            a = np.empty(n, np.float32)
            self._ok(fn(self.h, name.encode(), _ptr(a), n))
            out[name] = a
        return out

    def zero_grad(self):
        self._ok(self.L.gct_zero_grad(self.h))

    def set_lr(self, lr):
        self._ok(self.L.gct_set_lr(self.h, lr))

    def forward_backward(self, x, y, accum=1, want_loss=True, on_device=False):
        """x, y: [B, T] int64 (numpy / pinned torch host tensors, or CUDA tensors with on_device=True)."""
        B, T = x.shape
        loss = ctypes.c_float()
        self._ok(self.L.gct_forward_backward(self.h, _ptr(x), _ptr(y), 1 if on_device else 0, B, T, accum, ctypes.byref(loss) if want_loss else None))
        return loss.value if want_loss else None

    def optimizer_step(self, want_norm=False):
        norm = ctypes.c_float()
        self._ok(self.L.gct_optimizer_step(self.h, ctypes.byref(norm) if want_norm else None))
        return norm.value if want_norm else None

    def train_step(self, micro_batches, want_loss=True, on_device=False):
        """zero_grad, every micro-batch, clip + AdamW; returns the step loss (sum of the scaled micro-batch losses)."""
        self.zero_grad()
        tot = 0.0
        for x, y in micro_batches:
            l = self.forward_backward(x, y, len(micro_batches), want_loss, on_device)
            tot += l if want_loss else 0.0
        self.optimizer_step()
        return tot

    def generate(self, start_tokens, max_tokens, num_sequences=1, context_length=None, temperature=0.0, top_k=30):
        """[num_sequences, max_tokens] int64 token ids; argmax decoding unless temperature > 0."""
        import numpy as np

        start = np.ascontiguousarray(np.asarray(start_tokens, dtype=np.int64))
        out = np.zeros((num_sequences, max_tokens), dtype=np.int64)
        self._ok(self.L.gct_generate(self.h, _ptr(start), len(start), context_length or self.shape["T"], max_tokens, num_sequences, temperature, top_k, _ptr(out)))
        return out

    def save_checkpoint(self, model_path, optim_path):
        """Weights and AdamW state in the reference's checkpoint file format."""
        self._ok(self.L.gct_save_checkpoint(self.h, str(model_path).encode(), str(optim_path).encode()))

    def load_checkpoint(self, model_path, optim_path):
        self._ok(self.L.gct_load_checkpoint(self.h, str(model_path).encode(), str(optim_path).encode()))

    def sync(self):
        self._ok(self.L.gct_sync(self.h))

    def stream(self):
        return self.L.gct_stream(self.h)

    def context(self):
        return self.L.gct_context(self.h)

    def launch_count(self):
        return self.L.gct_launch_count(self.h)

    def high_water_bytes(self):
        return self.L.gct_arena_high_water_bytes(self.h)

    def num_buckets(self):
        return self.L.gct_num_buckets(self.h)

    def dp_init(self, unique_id, rank, world, accum_steps=1):
        self._ok(self.L.gct_dp_init(self.h, _ptr(unique_id), rank, world, accum_steps))

    def close(self):
        if self.h:
            self._ok(self.L.gct_destroy(self.h))
            self.h = None
