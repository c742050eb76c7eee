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
