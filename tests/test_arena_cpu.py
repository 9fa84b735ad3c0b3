"""Host side of the arena's crossing of process boundaries: the layout and descriptor protocol
over a unix socket (more descriptors than one message carries), the registry that manifests
consult, the load envelope's switch.  The reference tests its arena's host logic against a stub
backend in the same spirit (tests/test_vmm_arena.py); the device side is in the GPU tests."""

import os
import socket
import threading

import pytest

from modelexpress_b200 import arena as A


class FakeArena:
    """Stands in for an arena whose blocks are temp files: what travels is real descriptors."""

    def __init__(self, tmp_path, n_blocks, gran=2 << 20):
        self.device, self._h, self.base = 0, object(), 0x7000_0000_0000
        self.files = []
        for i in range(n_blocks):
            p = tmp_path / f"block{i}"
            p.write_bytes(f"block {i}".encode())
            self.files.append(str(p))
        self._blocks = [(i * gran, gran) for i in range(n_blocks)]
        self.used_bytes = n_blocks * gran

    def blocks(self):
        return list(self._blocks)

    def contains(self, ptr, nbytes=1):
        return self.base <= ptr and ptr + nbytes <= self.base + self.used_bytes

    def export_fds(self):
        fds = [os.open(f, os.O_RDONLY) for f in self.files]
        return {"device": 0, "span": self.used_bytes, "blocks": [list(b) for b in self._blocks]}, fds


@pytest.mark.parametrize("n_blocks", [0, 1, 7, 450])
def test_layout_and_descriptors_cross_a_socket(tmp_path, monkeypatch, n_blocks):
    fake = FakeArena(tmp_path, n_blocks)
    seen = {}

    def import_fds(cls, layout, fds, device):
        seen["layout"], seen["device"] = layout, device
        seen["content"] = [os.pread(fd, 64, 0).decode() for fd in fds]
        return "mapped"

    monkeypatch.setattr(A.Arena, "import_fds", classmethod(import_fds))
    path = str(tmp_path / "a.sock")
    server = A.ArenaServer(fake, path)
    try:
        before = len(os.listdir("/proc/self/fd"))
        assert A.fetch_arena(path, 3) == "mapped"
        assert A.fetch_arena(path, 3) == "mapped"     # every connection gets the current layout
        assert seen["device"] == 3 and seen["layout"]["span"] == fake.used_bytes
        assert seen["layout"]["blocks"] == [list(b) for b in fake.blocks()]
        assert seen["content"] == [f"block {i}" for i in range(n_blocks)]   # in order, none lost
        assert len(os.listdir("/proc/self/fd")) == before                   # both sides closed theirs
    finally:
        server.close()
    assert not os.path.exists(path)


def test_a_peer_that_hangs_up_is_an_error_not_a_hang(tmp_path):
    path = str(tmp_path / "b.sock")
    srv = socket.socket(socket.AF_UNIX, socket.SOCK_STREAM)
    srv.bind(path)
    srv.listen(1)

    def half():
        conn, _ = srv.accept()
        conn.sendall((100).to_bytes(8, "little") + b"{")   # announces 100 bytes, sends one, leaves
        conn.close()

    t = threading.Thread(target=half)
    t.start()
    with pytest.raises(ConnectionError):
        A.fetch_arena(path, 0, timeout_s=2.0)
    t.join()
    srv.close()


def test_registry_lookup_and_envelope_switch(tmp_path, monkeypatch):
    fake = FakeArena(tmp_path, 2)
    path = A.publish_arena(fake, str(tmp_path / "c.sock"))
    try:
        assert A.publish_arena(fake, path) == path                      # idempotent
        assert A.lookup(fake.base + 4096, 100) == (path, 4096)
        assert A.lookup(fake.base + fake.used_bytes - 10, 100) is None  # runs past the end
        assert A.lookup(0x1000, 16) is None
    finally:
        A.withdraw_arena(path)
    assert A.lookup(fake.base + 4096, 100) is None
    A.withdraw_arena(path)                                              # twice is fine
    monkeypatch.delenv("MXB_VMM_ARENA", raising=False)
    monkeypatch.delenv("MX_VMM_ARENA", raising=False)
    with A.maybe_enter_arena(0) as none:                                # unset: a no-op, no CUDA touched
        assert none is None
    monkeypatch.setenv("MX_VMM_ARENA", "1")
    assert A._env_on()
