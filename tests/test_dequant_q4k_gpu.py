"""Q4_K dequantization on the GPU: 0 ULP against the CPU checker, through the C ABI."""
import hashlib

import numpy as np
import pytest

from bpd_substrate_b200 import synth
from tests.util import Dev, assert_bits_equal

pytestmark = pytest.mark.gpu

SWEEP = ["dequant_v1_256", "dequant_v1_128", "dequant_v1_64", "dequant_v1_32",
         "dequant_ilp2", "dequant_multi2", "dequant_multi4", "dequant_multi8"]


def gpu_dequant(lib, q, nb, entry="bpd_dequant_q4k_gpu"):
    dq = Dev(lib, q)
    do = Dev(lib, nbytes=nb * 1024 + 64, fill=0x7F)   # poisoned, with a canary tail
    getattr(lib, entry)(dq.ptr, do.ptr, nb)
    lib.bpdq_sync()
    assert lib.bpdq_last_status() == 0
    raw = do.read(np.uint8)
    assert (raw[nb * 1024:] == 0x7F).all(), "wrote past the end of the output"
    return raw[:nb * 1024].view(np.float32)


@pytest.mark.parametrize("nb", [1, 2, 3, 63, 64, 65, 1000, 4096])
def test_bit_exact_random_blocks(lib, oracle, nb):
    q = synth.q4k_blocks(nb, 42 + nb)
    assert_bits_equal(gpu_dequant(lib, q, nb), oracle.dequant_q4k(q, 0))


def test_every_fp16_scale(lib, oracle):
    """All 65536 bit patterns of d and of dmin (subnormals, infinities and NaNs included)."""
    rng = np.random.default_rng(3)
    nb = 65536
    q = rng.integers(0, 256, size=(nb, 144), dtype=np.uint8)
    h = np.arange(nb, dtype=np.uint16)
    q[:, 0:2] = h.view(np.uint8).reshape(nb, 2)
    q[:, 2:4] = rng.permutation(h).view(np.uint8).reshape(nb, 2)
    q = q.reshape(-1)
    assert_bits_equal(gpu_dequant(lib, q, nb), oracle.dequant_q4k(q, 0))


@pytest.mark.parametrize("entry", SWEEP)
def test_sweep_shapes_write_whole_blocks(lib, oracle, entry):
    nb = 517  # not a multiple of 2, 4 or 8
    q = synth.q4k_blocks(nb, 9)
    assert_bits_equal(gpu_dequant(lib, q, nb, entry), oracle.dequant_q4k(q, 0))


@pytest.mark.parametrize("entry", ["run_bpd", "run_llamacpp"])
def test_ggml_nibble_order(lib, oracle, entry):
    nb = 4096
    q = synth.q4k_blocks(nb, 17)
    got = gpu_dequant(lib, q, nb, entry)
    assert_bits_equal(got, oracle.dequant_q4k(q, 1))
    assert not np.array_equal(got, oracle.dequant_q4k(q, 0))


def test_zero_blocks_is_a_no_op(lib):
    lib.bpd_dequant_q4k_gpu(None, None, 0)
    assert lib.bpdq_last_status() == 0


def test_full_tensor_14336x4096(lib, oracle):
    """The whole benchmark tensor (229,376 super-blocks): 0 ULP on all 58,720,256 outputs."""
    nb = 14336 * 16
    q = synth.q4k_blocks(nb, 1000)
    got = gpu_dequant(lib, q, nb)
    want = oracle.dequant_q4k(q, 0)
    assert hashlib.sha256(got.tobytes()).hexdigest() == hashlib.sha256(want.tobytes()).hexdigest()


def test_full_tensor_against_reference_fixture(lib):
    """Same tensor against the fixture written by the reference's own C code (hash + samples)."""
    import os
    g = np.load(os.path.join(os.path.dirname(__file__), "golden", "q4k_dequant_14336x4096.npz"))
    nb = int(g["n_blocks"][0])
    q = synth.q4k_blocks(nb, int(g["seed"][0]))
    got = gpu_dequant(lib, q, nb)
    assert hashlib.sha256(got.tobytes()).hexdigest() == str(g["output_sha256"][0])
    assert np.array_equal(got[::int(g["sample_stride"][0])].view(np.uint32), g["sample"])


def test_small_fixture_from_reference(lib):
    import os
    g = np.load(os.path.join(os.path.dirname(__file__), "golden", "q4k_small.npz"))
    got = gpu_dequant(lib, g["q"], g["q"].size // 144)
    assert np.array_equal(got.view(np.uint32), g["dequant"])
