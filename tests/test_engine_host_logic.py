"""CPU: host-side logic of the Engine mirror that needs no GPU — the prepared-input cache policy
of the reference (src/inference.hpp:221-289) and which host objects may be cached at all."""
import numpy as np

from munet_b200.inference import PreparedInputCache, _input_identity


def test_cache_limits_and_eviction_order():
    c = PreparedInputCache(max_entries=2, max_bytes=100)
    assert c.store("a", 0, "A", 40) == 0 and c.store("b", 0, "B", 40) == 0
    assert len(c) == 2 and c.current_bytes == 80
    assert c.find("a", 0) == "A" and c.find("a", 1) is None      # a newer version is a miss
    assert c.store("c", 0, "C", 40) == 1                          # entry limit: the oldest goes
    assert c.find("a", 0) is None and c.find("b", 0) == "B" and c.find("c", 0) == "C"
    assert c.store("d", 0, "D", 90) == 2                          # byte limit: evict until it fits
    assert len(c) == 1 and c.current_bytes == 90
    assert c.store("e", 0, "E", 101) == 0 and len(c) == 1         # larger than the cache: not stored
    assert c.store("d", 5, "D2", 10) == 0                         # same identity: replaced in place
    assert c.find("d", 0) is None and c.find("d", 5) == "D2" and c.current_bytes == 10
    c.configure(0, 100)
    assert c.store("x", 0, "X", 1) == 0 and len(c) == 0           # disabled


def test_only_inputs_whose_changes_can_be_seen_are_cached():
    a = np.zeros((2, 3), np.float32)
    assert _input_identity(a) is None                              # writable numpy: no version
    a.flags.writeable = False
    assert _input_identity(a) is not None
    import torch
    t = torch.zeros(2, 3)
    k0 = _input_identity(t)
    t.add_(1.0)
    k1 = _input_identity(t)
    assert k0[0] == k1[0] and k1[1] == k0[1] + 1                   # in-place op bumps the version


def test_attention_size_checks_do_not_wrap():
    """Sizes whose product B*H*T*T*sizeof wraps in 64 bits (2^64 here) must be refused, not taken
    for zero bytes. Nothing is launched on these paths, so no GPU is needed."""
    import ctypes as C
    import munet_b200 as mb
    lib = mb.lib()
    err = C.create_string_buffer(512)
    dummy = 0x1000  # never dereferenced: the size check comes first
    rc = lib.mu_attention_static_scratch(0, dummy, dummy, dummy, dummy, 32768, 32768, 65536, 16, 1, 0, 0,
                                         None, 0, err, 512)
    assert rc == 7 and b"exceed" in err.value                     # MU_ERR_SIZE
    rc = lib.mu_attention_static_scratch(0, dummy, dummy, dummy, dummy, 1, 1, 8192, 16, 1, 0, 0,
                                         None, 0, err, 512)
    assert rc == 7                                                # 256 MiB of scores > 64 MiB
    assert lib.mu_attention_workspace_bytes_composed(32768, 32768, 65536, 16, 0) == 0
    assert lib.mu_attention_workspace_bytes(32768, 32768, 65536, 16, 0) == 0
    assert lib.mu_attention_workspace_bytes_composed(2, 3, 40, 16, 0) == 2 * 3 * 40 * 40 * 4
    assert lib.mu_attention_workspace_bytes(2, 16, 1024, 128, 2) == 0   # fused kernel: no workspace
    assert lib.mu_attention_workspace_bytes_composed(2, 16, 1024, 128, 2) == 2 * 16 * 1024 * 1024 * 2


def test_host_inputs_are_converted_to_the_compiled_dtype():
    """What run() and prepare_batch() hand to the engine: values converted to the compiled input
    dtype (torch.randint's int64 ids, float64 arrays), 16-bit patterns for a bfloat16 input taken
    as bits."""
    import torch
    import oracle
    from munet_b200.inference import _as_host_tensor
    from munet_b200 import BF16, F32, I32
    ids = torch.randint(0, 1000, (2, 5))
    t = _as_host_tensor(ids, I32)
    assert t.dtype == torch.int32 and torch.equal(t.long(), ids) and t.is_contiguous()
    t = _as_host_tensor(np.arange(6, dtype=np.float64).reshape(2, 3) / 3, F32)
    assert t.dtype == torch.float32 and np.allclose(t.numpy(), np.arange(6).reshape(2, 3) / 3)
    bits = oracle.to_bf16(np.array([1.0, -2.5, 3.25], np.float32))
    t = _as_host_tensor(bits, BF16)
    assert t.dtype == torch.bfloat16 and t.float().tolist() == [1.0, -2.5, 3.25]
    t = _as_host_tensor(torch.from_numpy(bits.view(np.int16)), BF16)
    assert t.float().tolist() == [1.0, -2.5, 3.25]
    t = _as_host_tensor(torch.tensor([1.0, -2.5]), BF16)          # float32 values -> bf16 by value
    assert t.dtype == torch.bfloat16 and t.float().tolist() == [1.0, -2.5]
    nc = torch.arange(12, dtype=torch.int32).reshape(3, 4).t()    # non-contiguous view
    assert _as_host_tensor(nc, I32).is_contiguous()
