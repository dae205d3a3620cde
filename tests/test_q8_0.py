"""The first narrow weight form, Q8_0 (engine/ir/mem/src/block.rs:259-260).

CPU part: the checker's restatement of the form is pinned to the reference's own test
(engine/ir/mem/src/block_test.rs:7-56, `blocks_round_trip`: its data, its sizes, its bounds), and the library's
host-side packer must produce the checker's bytes.  GPU part: ts_linear_q8_0 against the checker's matmul over the
same packed bytes.  Tolerance 1e-2 of the largest output for bf16 outputs, 1e-4 for f32 (the codes are exact in the
tensor-core operands, so only the order of the f32 sums differs)."""
import ctypes as C

import numpy as np
import pytest
import torch

import oracle as O


def _reference_data(n=128):
    return np.array([((i * 37) % 23) * 0.01 - 0.1 for i in range(n)], np.float32)


def test_oracle_follows_blocks_round_trip():
    data = _reference_data()
    packed = O.q8_0_pack(data)
    assert packed.size == 136                                   # form.bytes(128)
    back = O.q8_0_unpack(packed, 128)
    top = float(np.abs(data).max())
    assert float(np.abs(back - data).max()) <= top * 0.005      # Q8_0's share in the reference's table
    x = np.array([(i % 7) - 3.0 for i in range(128)], np.float32)
    want = float(np.sum(x * back, dtype=np.float32))
    got = float(O.matmul_q8_0(x[None], packed, 1)[0, 0])
    assert abs(got - want) <= 1e-4                              # "a dot matches the plain sum over the unpacked elements"
    assert O.q8_0_pack(np.zeros(64, np.float32)).size == 68     # Q8_0.bytes(64)
    # a block's largest value lands on code +-127 and the scale is its f16 rounding
    block = np.zeros(32, np.float32)
    block[3], block[9] = -0.5, 0.25
    b = O.q8_0_pack(block)
    assert np.frombuffer(b[:2].tobytes(), np.float16)[0] == np.float16(0.5 / 127)
    assert b[2 + 3].astype(np.int8) == -127 and abs(int(b[2 + 9].astype(np.int8)) - 64) <= 1


def test_library_packer_writes_the_checkers_bytes():
    from tessera_b200 import _lib
    rng = np.random.default_rng(2)
    for n in (32, 128, 4096, 100):                              # 100: a ragged last block
        data = (rng.standard_normal(n) * 0.02).astype(np.float32)
        data[: min(n, 40)] *= 50.0
        if n >= 64:
            data[32:64] = 0.0                                   # an all-zero block: scale 0, codes 0
        size = _lib.lib.ts_q8_0_bytes(n)
        out = np.zeros(size, np.uint8)
        _lib.check(_lib.lib.ts_q8_0_pack(data.ctypes.data_as(C.c_void_p), n, out.ctypes.data_as(C.c_void_p)))
        assert np.array_equal(out, O.q8_0_pack(data))
        back = np.empty(n, np.float32)
        _lib.check(_lib.lib.ts_q8_0_unpack(out.ctypes.data_as(C.c_void_p), n, back.ctypes.data_as(C.c_void_p)))
        assert np.array_equal(back, O.q8_0_unpack(out, n))


def test_sizes_the_kernel_does_not_take_are_refused():
    from tessera_b200 import _lib
    buf = (C.c_char * 4096)()
    p = (C.cast(buf, C.c_void_p).value + 15) // 16 * 16
    for m, n, k in ((65, 64, 256), (4, 48, 256), (4, 64, 128)):
        rc = _lib.lib.ts_linear_q8_0(p, p, None, p, m, n, k, 0, 1.0, 0, p, 4096, None)
        assert rc == _lib.TS_ERR_BAD_INPUT and b"q8_0" in _lib.lib.ts_last_error()


@pytest.mark.gpu
@pytest.mark.parametrize("m,n,k", [(1, 64, 256), (7, 1024, 1024), (64, 4096, 1024), (64, 1024, 3072), (33, 6144, 1024),
                                   (64, 192, 512)])
def test_linear_matches_oracle(m, n, k):
    from tessera_b200 import ops
    from tests.util import from_bits, normal_bf16, rel_error, widen
    rng = np.random.default_rng(m + n + k)
    x = normal_bf16(rng, (m, k))
    w = (rng.standard_normal((n, k)) * 0.02).astype(np.float32)
    packed = O.q8_0_pack(w)
    want = O.matmul_q8_0(O.bf16_widen(x), packed, n)
    wq = torch.from_numpy(packed.reshape(n, k // 32 * 34)).cuda()
    assert torch.equal(ops.q8_0_pack(torch.from_numpy(w)).cpu(), wq.cpu())
    got32 = ops.linear_q8_0(from_bits(x), wq, out_dtype=torch.float32)
    got16 = ops.linear_q8_0(from_bits(x), wq)
    again = ops.linear_q8_0(from_bits(x), wq, out_dtype=torch.float32)
    torch.cuda.synchronize()
    assert rel_error(widen(got32), want) <= 1e-4
    assert rel_error(widen(got16), want) <= 1e-2
    assert torch.equal(got32, again)                            # slices add in a fixed order


@pytest.mark.gpu
def test_fused_epilogues():
    from tessera_b200 import ops
    from tests.util import from_bits, normal_bf16, rel_error, widen
    rng = np.random.default_rng(9)
    m, ffn, k = 40, 768, 512
    x = normal_bf16(rng, (m, k))
    w = (rng.standard_normal((2 * ffn, k)) * 0.05).astype(np.float32)
    packed = O.q8_0_pack(w)
    wq = torch.from_numpy(packed.reshape(2 * ffn, k // 32 * 34)).cuda()
    full = O.matmul_q8_0(O.bf16_widen(x), packed, 2 * ffn)
    want = O.act(full[:, :ffn], "silu") * full[:, ffn:]
    got = ops.linear_q8_0(from_bits(x), wq, epilogue="swiglu")
    res = rng.standard_normal((m, 2 * ffn), dtype=np.float32)
    added = ops.linear_q8_0(from_bits(x), wq, torch.from_numpy(res).cuda(), epilogue="add", out_dtype=torch.float32)
    torch.cuda.synchronize()
    assert rel_error(widen(got), want) <= 1e-2
    assert rel_error(widen(added), full + res) <= 1e-4
