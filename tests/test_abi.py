"""CPU-side checks of the C-ABI library: it builds, loads, exports every symbol the header declares, and
argument validation answers with status codes (no kernel is launched here)."""

import ctypes as C

import pytest

from emmy_b200 import lib as L


@pytest.fixture(scope="module")
def eq():
    from emmy_b200.build import build

    build()
    return L.load()


def test_exports_every_declared_symbol(eq):
    names = L.declared_symbols()
    assert len(names) >= 12
    for name in names:
        assert hasattr(eq, name), f"libemmyq.so does not export {name}"
    assert set(names) == set(eq._eq_signatures), "lib.py binds a different set of symbols than the header declares"


def test_version_and_status_names(eq):
    assert eq.eq_version() >= 100
    assert eq.eq_status_name(0) == b"EQ_OK"
    assert eq.eq_status_name(L.EQ_ERR_WORKSPACE) == b"EQ_ERR_WORKSPACE"
    assert eq.eq_status_name(-99) == b"EQ_ERR_UNKNOWN"


def test_bad_arguments_return_codes_not_crashes(eq):
    null = C.c_void_p(0)
    one = C.c_void_p(16)  # never dereferenced: validation fails first
    assert eq.eq_unpack_int4(7, 0, one, 1, 1, one, null) == L.EQ_ERR_BAD_ARG
    assert eq.eq_unpack_int4(0, 0, null, 1, 1, one, null) == L.EQ_ERR_BAD_ARG
    assert b"null" in eq.eq_last_error()
    # group geometry that does not cover K (the reference raises ValueError: quant.py:546-547)
    assert eq.eq_dequant_w4(0, one, one, one, 0, null, 256, 64, 100, 0, 0, one, null) == L.EQ_ERR_BAD_ARG
    assert eq.eq_dequant_fp8(one, one, 16, 64, 3, 1, 2, one, null) == L.EQ_ERR_BAD_ARG
    assert eq.eq_dequant_nvfp4(one, one, one, 4, 20, 2, one, null) == L.EQ_ERR_BAD_ARG
    a = C.c_size_t()
    assert eq.eq_w4_repack_sizes(100, 64, 128, C.byref(a), None) == L.EQ_ERR_BAD_ARG
    assert eq.eq_w4_repack_sizes(4096, 4096, 32, C.byref(a), None) == L.EQ_ERR_UNSUPPORTED
    assert eq.eq_w4_repack_sizes(4096, 4096, 128, C.byref(a), None) == 0 and a.value == 256 * 32 * 1088
    # linear: workspace too small, misaligned weights
    assert eq.eq_w4a16_linear(one, 0, null, 4096, 4096, 128, one, 1, 0, one, null, 0, null) == L.EQ_ERR_WORKSPACE
    assert eq.eq_w4a16_linear(C.c_void_p(8), 0, null, 4096, 4096, 128, one, 1, 0, one, one, 1 << 20, null) == L.EQ_ERR_BAD_ALIGN
    assert eq.eq_w4a16_linear(one, 0, null, 4096, 4096, 128, one, 1, 2, one, one, 1 << 20, null) == L.EQ_ERR_BAD_ARG
    assert eq.eq_w4a16_linear(one, 0, null, 4096, 4096, 64, one, 1, 0, one, one, 1 << 20, null) == L.EQ_ERR_UNSUPPORTED
    # the allocation-free variant validates before anything else, also for an empty call
    assert eq.eq_w4a16_linear_noalloc(one, 0, null, 4096, 4096, 64, one, 0, 0, one, null) == L.EQ_ERR_UNSUPPORTED
    assert eq.eq_w4a16_linear_noalloc(one, 0, null, 4096, 4096, 128, one, 0, 5, one, null) == L.EQ_ERR_BAD_ARG
    assert eq.eq_w4a16_linear_noalloc(one, 0, null, 4096, 65536, 128, one, 1, 0, one, null) == L.EQ_ERR_UNSUPPORTED
    # a 256-byte header (status word first), f32 words, one counter per 16-column tile
    assert eq.eq_w4a16_workspace_bytes(1, 4096, 4096) == 256 + 4096 * 4 + 256 * 4
    front = 256 + 100 * 4096 * 4 + 256 * 4
    assert eq.eq_w4a16_workspace_bytes(100, 4096, 256) == (front + 255) // 256 * 256 + 100 * 256 * 2


def test_peer_allreduce_validates_before_it_launches(eq):
    null = C.c_void_p(0)
    one = C.c_void_p(16)  # never dereferenced: validation fails first
    peers = L.ArPeers()
    peers.world, peers.rank, peers.cap, peers.max_blocks = 2, 0, 4096, 2
    for r in range(2):
        peers.recv[r], peers.flags[r] = 16, 16
    ok = lambda count, dtype=L.EQ_F16, y=one: eq.eq_peer_allreduce(C.byref(peers), one, count, dtype, y, one, null)
    assert ok(0) == 0                                   # an empty call does nothing
    assert ok(12) == L.EQ_ERR_UNSUPPORTED               # whole 16-byte vectors only
    assert ok(4104) == L.EQ_ERR_UNSUPPORTED             # more than the buffers carry
    assert ok(8, dtype=L.EQ_F32) == L.EQ_ERR_BAD_ARG    # f16 / bf16 partials
    assert ok(8, y=C.c_void_p(8)) == L.EQ_ERR_BAD_ALIGN
    peers.max_blocks = 3
    assert ok(8) == L.EQ_ERR_BAD_ARG                    # the flag layout must match the capacity
    peers.max_blocks, peers.rank = 2, 2
    assert ok(8) == L.EQ_ERR_BAD_ARG
    assert eq.eq_peer_allreduce_recv_bytes(8, 64 * 4096) == 2 * 8 * 64 * 4096 * 2
    assert eq.eq_peer_allreduce_flag_bytes(8, 64 * 4096) == 2 * 8 * 128 * 4
    assert eq.eq_peer_allreduce_state_bytes() >= 12


def test_ops_refuse_cpu_tensors():
    torch = pytest.importorskip("torch")
    from emmy_b200 import ops

    with pytest.raises(RuntimeError, match="no CPU path"):
        ops.unpack_int4(torch.zeros(2, 2, dtype=torch.int32), "awq")
