"""The reference's own ctypes ABI served by this library (include/flyvec_ref_abi.h): the symbols exist
under the reference's five library names, and -- on a GPU -- the exact call sequence of the reference's
driver (flyvec/train_flyvec.py:141-263) trains a model that equals the one the fv_* API produces."""
import ctypes
import os
import re
from ctypes import c_char_p, c_float, c_int32, c_uint64, c_void_p
from pathlib import Path

import numpy as np
import pytest

from flyvec_b200 import _lib, synth
from flyvec_b200.engine import Trainer

HEADER = Path(__file__).resolve().parent.parent / "include" / "flyvec_ref_abi.h"


def ref_names():
    text = re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.S)
    return sorted(set(re.findall(r"\b([a-zA-Z_][a-zA-Z0-9_]*)\s*\(", text)) - {"defined"})


def test_reference_symbols_are_exported(built_lib):
    names = ref_names()
    assert len(names) == 24
    for n in names:
        assert hasattr(built_lib, n), n
    d = _lib.make_ref_abi_links()
    for so in _lib.REF_ABI_NAMES:
        assert (d / so).resolve() == _lib.LIB_PATH.resolve()


#: the library calls of the reference driver's ``main`` in source order, runs of the same call collapsed
#: (flyvec/train_flyvec.py:141-263)
DRIVER_CALLS = ["get_cuda_num_devices", "model_create_descriptor", "model_create_arrays", "do_gpu_cudaHostAlloc",
                "getnum_samples", "do_gpu_cudaHostAlloc", "compute_offset_phrases", "print_model_params",
                "set_model_param_int", "set_model_param_float", "compute_model_derived_parameters", "copy_model_params",
                "print_model_params", "model_arrays_allocate_memory", "set_up_INPUT_pointer",
                "compute_inverse_word_frequency", "get_data_pointer", "do_reshuffle_indices", "launch_epoch_INPUT_AS_INT"]


def collapse(seq):
    return [c for i, c in enumerate(seq) if i == 0 or seq[i - 1] != c]


def test_replayed_sequence_is_the_reference_drivers():
    """The call sequence the GPU test below replays is read off the reference's own driver: its ``main``
    is parsed (not imported) and every call into one of the five libraries, direct or through the
    ``py_*`` aliases, is listed in source order."""
    import ast

    from oracle.build_oracle import reference_root

    ref = reference_root()
    if ref is None:
        pytest.skip("no reference checkout")
    tree = ast.parse((ref / "flyvec" / "train_flyvec.py").read_text())
    main = [n for n in tree.body if isinstance(n, ast.FunctionDef) and n.name == "main"][0]
    libs = {"model_descriptor", "model_arrays", "cuda_helpers", "model", "prune_input"}
    alias, seq = {}, []

    class Walk(ast.NodeVisitor):
        def visit_Assign(self, node):
            v = node.value
            if (isinstance(v, ast.Attribute) and isinstance(v.value, ast.Name) and v.value.id in libs
                    and len(node.targets) == 1 and isinstance(node.targets[0], ast.Name)):
                alias[node.targets[0].id] = v.attr
            self.generic_visit(node)

        def visit_Call(self, node):
            f = node.func
            if isinstance(f, ast.Name) and f.id in alias:
                seq.append(alias[f.id])
            elif isinstance(f, ast.Attribute) and isinstance(f.value, ast.Name) and f.value.id in libs:
                seq.append(f.attr)
            self.generic_visit(node)

    Walk().visit(main)
    assert collapse(seq) == DRIVER_CALLS
    assert set(seq) <= set(ref_names())


class Recording:
    """A CDLL whose calls are logged by name."""

    def __init__(self, lib, log):
        self._lib, self._log = lib, log

    def __getattr__(self, name):
        fn = getattr(self._lib, name)

        def call(*a):
            self._log.append(name)
            return fn(*a)

        call.fn = fn
        return call


@pytest.mark.gpu
def test_reference_driver_call_sequence(built_lib, tmp_path, monkeypatch):
    """Replays train_flyvec.py's calls, with its own argument wrappers, on a small corpus, and compares
    the checkpoint it leaves with the oracle's epochs over the same window order."""
    from oracle import flyvec_oracle as orc
    from tests.test_gpu_shapes import assert_weights_close

    monkeypatch.setenv("FLYVEC_SEED", "5")
    BIN = _lib.make_ref_abi_links()
    log = []
    raw = {n: ctypes.CDLL(str(BIN / f"{n}.so")) for n in ("model_descriptor", "model_arrays", "cuda_helpers", "cuda_funcs", "prune_input")}
    raw["model_descriptor"].model_create_descriptor.restype = c_void_p
    raw["model_arrays"].model_create_arrays.restype = c_void_p
    raw["cuda_helpers"].do_gpu_cudaHostAlloc.restype = c_void_p
    raw["model_arrays"].get_data_pointer.restype = c_void_p
    raw["prune_input"].getnum_samples.restype = c_uint64
    model_descriptor, model_arrays = Recording(raw["model_descriptor"], log), Recording(raw["model_arrays"], log)
    cuda_helpers, model, prune_input = Recording(raw["cuda_helpers"], log), Recording(raw["cuda_funcs"], log), Recording(raw["prune_input"], log)

    W, hid, batch_size, lr, Nep = 7, 48, 300, 0.002, 2
    enc, off = synth.make_corpus(20000, 300, mean_len=20, min_len=W, seed=3)
    num_gpus = cuda_helpers.get_cuda_num_devices()
    assert num_gpus == 1
    DSCR = model_descriptor.model_create_descriptor(c_int32(num_gpus))
    DATA = model_arrays.model_create_arrays(c_int32(num_gpus))
    Ns_1 = enc.shape[0]
    INPUT = cuda_helpers.do_gpu_cudaHostAlloc(c_uint64(Ns_1 * 4))
    inp = np.ctypeslib.as_array(ctypes.cast(INPUT, ctypes.POINTER(ctypes.c_int32)), shape=(Ns_1,))
    np.copyto(inp, enc)
    V = int(inp.max()) + 1
    N = 2 * V
    nsent = off.shape[0] - 1
    nphr = prune_input.getnum_samples(c_void_p(off.ctypes.data), c_uint64(nsent), c_uint64(W))
    PHR = cuda_helpers.do_gpu_cudaHostAlloc(c_uint64((nphr + 1) * 8))
    prune_input.compute_offset_phrases(c_void_p(PHR), c_void_p(off.ctypes.data), c_uint64(nsent), c_uint64(W))
    model_descriptor.print_model_params(c_void_p(DSCR))
    for k, v in ((b"IM_HEIGHT", 1), (b"IM_WIDTH", 11), (b"Nchannels", 1), (b"Ns_1", c_uint64(nphr)), (b"W", W), (b"ST", 1),
                 (b"hid", hid), (b"Num", batch_size), (b"vocabulary_size", c_uint64(V)), (b"sparse_input", 1),
                 (b"frequency_scaling", 1)):
        model_descriptor.set_model_param_int(v, k, c_void_p(DSCR))
    for k, v in ((b"initial_learning_rate", lr), (b"delta", 0.0), (b"prec", 1e-30), (b"mu", 0.0), (b"sigma", 0.02),
                 (b"Lmid", 1.0), (b"Lbase", 1.0)):
        model_descriptor.set_model_param_float(c_float(v), k, c_void_p(DSCR))
    model_descriptor.compute_model_derived_parameters(c_void_p(DSCR))
    for gpu in range(1, num_gpus):
        model_descriptor.copy_model_params(c_void_p(DSCR), c_int32(0), c_int32(gpu))
    model_descriptor.print_model_params(c_void_p(DSCR))
    model_arrays.model_arrays_allocate_memory(c_void_p(DSCR), c_void_p(DATA), c_int32(num_gpus))
    model_arrays.set_up_INPUT_pointer(b"INPUT", c_void_p(DATA), c_void_p(DSCR), c_void_p(INPUT), c_void_p(PHR), b"i4",
                                      c_int32(0))
    model_arrays.compute_inverse_word_frequency(c_void_p(DATA), c_void_p(DSCR), c_void_p(INPUT), c_uint64(Ns_1), c_int32(0))
    R = synth.make_weights(hid, N, seed=4, sigma=0.5)
    syn_ptr = ctypes.cast(model_arrays.get_data_pointer(b"synapses", c_void_p(DATA), c_int32(0)), ctypes.POINTER(ctypes.c_float))
    syn = np.ctypeslib.as_array(syn_ptr, shape=(hid, N))
    np.copyto(syn, R)
    for ep in range(Nep):
        model_arrays.do_reshuffle_indices(c_void_p(DSCR), c_void_p(DATA), c_int32(0))
        model.launch_epoch_INPUT_AS_INT(c_void_p(DSCR), c_void_p(DATA), c_int32(num_gpus), c_uint64(ep), c_uint64(Nep))
        np.save(tmp_path / f"ckpt_{ep}", syn)
    got = np.load(tmp_path / f"ckpt_{Nep - 1}.npy")
    # the replay made the driver's calls in the driver's order (copy_model_params only runs with several GPUs)
    assert collapse(log) == [c for c in DRIVER_CALLS if c != "copy_model_params"][:-2] + ["do_reshuffle_indices", "launch_epoch_INPUT_AS_INT"] * Nep

    tr = Trainer(hid=hid, vocab=V, window=W, batch=batch_size, lr0=lr, flags=_lib.FV_FLAG_COUNT_FP32)
    assert tr.set_corpus(enc, off) == nphr
    tr.set_weights(R)
    for ep in range(Nep):
        tr.shuffle(5 * 1000003 + ep)
        tr.run_epoch(ep, Nep)
        tr.set_weights(tr.get_weights())  # the shim round-trips the weights through the host slab every epoch
    want = tr.get_weights()
    np.testing.assert_array_equal(got, want)
    assert np.abs(got - R).max() > 1e-4
    # and against the oracle: the same epochs over the window orders the library drew
    starts = orc.enumerate_windows(off, W)
    f = orc.inverse_word_frequency(enc, V, saturate_fp32=True)
    Wref = R
    for ep in range(Nep):
        tr.shuffle(5 * 1000003 + ep)
        Wref, _ = orc.run_epoch(Wref, enc, starts, tr.get_permutation(), f, V, W, batch_size, 1, orc.epoch_eps(lr, ep, Nep))
    tr.close()
    assert_weights_close(got, Wref)
