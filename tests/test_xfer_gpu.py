"""The binding's host <-> device copies (seedpack_b200.refbind.xfer): chunked copies through the worker threads' page-locked
slots must move exactly the bytes a plain copy moves - sizes around the chunk and hand-over limits, sources that are
read-only or start at odd addresses, destinations that are views of larger arrays, page-locked arrays (copied directly),
and several copies in flight from different threads."""
import threading

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _sizes(x):
    return [0, 1, 4095, x.DIRECT - 1, x.DIRECT, x.DIRECT + 1, x.CHUNK - 3, x.CHUNK, x.CHUNK + 17, 3 * x.CHUNK + 12345]


def test_uploads_and_downloads_move_the_same_bytes():
    from seedpack_b200.refbind import xfer
    rng = np.random.default_rng(3)
    big = rng.integers(0, 256, 3 * xfer.CHUNK + 12345 + 64, dtype=np.uint8)
    for n in _sizes(xfer):
        for lead in (0, 1, 13):                                   # odd start addresses on the host side
            src = big[lead:lead + n]
            dev = torch.empty(n + 32, dtype=torch.uint8, device="cuda")[16:16 + n] if n else torch.empty(0, dtype=torch.uint8, device="cuda")
            if n:
                xfer.h2d(dev, src)
                assert torch.equal(dev.cpu(), torch.from_numpy(src.copy())), (n, lead)
                back = np.zeros(n + 9, np.uint8)
                xfer.d2h(back[7:7 + n], dev)
                assert np.array_equal(back[7:7 + n], src) and back[:7].sum() == 0 and back[7 + n:].sum() == 0, (n, lead)


def test_read_only_and_page_locked_hosts():
    from seedpack_b200.refbind import xfer
    n = xfer.CHUNK + 4097
    raw = bytes(np.random.default_rng(4).integers(0, 256, n, dtype=np.uint8))
    ro = np.frombuffer(raw, np.uint8)                            # read-only: a file's bytes
    dev = torch.empty(n, dtype=torch.uint8, device="cuda")
    xfer.h2d(dev, ro)
    assert dev.cpu().numpy().tobytes() == raw
    pinned = torch.empty(n, dtype=torch.uint8, pin_memory=True).numpy()
    xfer.d2h(pinned, dev)                                        # page-locked destination: one direct copy
    assert pinned.tobytes() == raw
    dev2 = torch.empty(n, dtype=torch.uint8, device="cuda")
    xfer.h2d(dev2, pinned)
    assert torch.equal(dev, dev2)


def test_copies_from_several_threads_at_once():
    from seedpack_b200.refbind import xfer
    n = 2 * xfer.CHUNK + 999
    srcs = [np.full(n, k + 1, np.uint8) for k in range(4)]
    devs = [torch.empty(n, dtype=torch.uint8, device="cuda") for _ in srcs]
    errs = []

    def one(k):
        try:
            torch.cuda.set_device(0)
            xfer.h2d(devs[k], srcs[k])
            out = np.zeros(n, np.uint8)
            xfer.d2h(out, devs[k])
            if not np.array_equal(out, srcs[k]):
                errs.append(k)
        except Exception as e:                                  # noqa: BLE001
            errs.append(repr(e))

    ts = [threading.Thread(target=one, args=(k,)) for k in range(4)]
    for t in ts:
        t.start()
    for t in ts:
        t.join()
    assert not errs, errs
