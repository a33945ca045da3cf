"""The registry of device twins (seedpack_b200.refbind.twins) as host logic: look-ups by address range, sub-views,
release with the owning array, replacement at a reused address, eviction beyond the byte cap.  The "device" tensors
here are CPU tensors: the registry only stores and slices them."""
import gc

import numpy as np
import torch

from seedpack_b200.refbind import twins


def _pair(n, fill):
    h = np.full(n, fill, np.uint8)
    return h, torch.from_numpy(h.copy())


def setup_function(_):
    twins.clear()


def test_views_find_their_slice_and_strangers_find_nothing():
    h, d = _pair(4096, 7)
    twins.register(h, d)
    v = h[100:356]
    t = twins.find(v)
    assert t is not None and t.numel() == 256 and t.data_ptr() == d.data_ptr() + 100
    assert twins.find(h.view(np.uint16)[8:24]).numel() == 32          # other element types: bytes are what counts
    assert twins.find(np.zeros(16, np.uint8)) is None                 # an array that was never registered
    assert twins.find(h[::2]) is None                                 # not contiguous
    big = np.zeros(8192, np.uint8)
    twins.register(big[:1024], torch.zeros(1024, dtype=torch.uint8))
    assert twins.find(big[512:2048]) is None                          # reaches past the registered range


def test_entry_goes_with_the_array_that_owns_the_memory():
    h, d = _pair(1 << 16, 1)
    view = h[:1024]
    twins.register(view, d[:1024])                                     # registered through a view: the owner is h
    del view
    gc.collect()
    assert twins.find(h[:16]) is not None
    addr = h.__array_interface__["data"][0]
    del h
    gc.collect()
    assert addr not in twins._ents and not twins._starts


def test_registering_again_at_the_same_address_replaces():
    h, d1 = _pair(2048, 3)
    twins.register(h, d1)
    d2 = torch.full((2048,), 9, dtype=torch.uint8)
    twins.register(h, d2)
    assert int(twins.find(h[:4])[0]) == 9
    assert twins._bytes[0] == 2048 and len(twins._starts) == 1


def test_oldest_entries_leave_when_the_cap_is_passed(monkeypatch):
    monkeypatch.setattr(twins, "CAP", 3000)
    keep = [_pair(1024, k) for k in range(5)]
    for h, d in keep:
        twins.register(h, d)
    assert twins._bytes[0] <= 3000 + 1024
    assert twins.find(keep[0][0]) is None and twins.find(keep[1][0]) is None      # the oldest went
    assert twins.find(keep[4][0]) is not None and twins.find(keep[3][0]) is not None
