"""The Redis storage plugin of the dynamic-embedding library against an in-test RESP server: evict -> fetch round trip through
MSET / MGET, unknown ids, key prefix, server gone."""
import os
import socketserver
import threading

import pytest
import torch

from torchrec_b200.ops import _ext

PLUGIN = os.path.join(os.path.dirname(_ext.CPU_LIB_PATH), "_tde_redis_io.so")
pytestmark = pytest.mark.skipif(not (_ext.has_cpu_ext() and os.path.exists(PLUGIN)), reason="native libraries not built")


class _FakeRedis(socketserver.ThreadingTCPServer):
    allow_reuse_address = True
    daemon_threads = True

    def __init__(self):
        self.kv = {}
        self.commands = []
        self.lock = threading.Lock()
        super().__init__(("127.0.0.1", 0), _Handler)


class _Handler(socketserver.StreamRequestHandler):
    def _read_command(self):
        head = self.rfile.readline()
        if not head:
            return None
        assert head[:1] == b"*", head
        args = []
        for _ in range(int(head[1:].strip())):
            n = int(self.rfile.readline()[1:].strip())
            args.append(self.rfile.read(n))
            self.rfile.read(2)
        return args

    def handle(self):
        srv = self.server
        while True:
            try:
                cmd = self._read_command()
            except Exception:
                return
            if cmd is None:
                return
            name = cmd[0].upper()
            with srv.lock:
                srv.commands.append(name)
                if name == b"MSET":
                    for k, v in zip(cmd[1::2], cmd[2::2]):
                        srv.kv[k] = v
                    self.wfile.write(b"+OK\r\n")
                elif name == b"MGET":
                    out = b"*%d\r\n" % (len(cmd) - 1)
                    for k in cmd[1:]:
                        v = srv.kv.get(k)
                        out += b"$-1\r\n" if v is None else b"$%d\r\n%s\r\n" % (len(v), v)
                    self.wfile.write(out)
                elif name in (b"SELECT", b"PING"):
                    self.wfile.write(b"+OK\r\n")
                else:
                    self.wfile.write(b"-ERR unknown command\r\n")


@pytest.fixture(scope="module")
def redis():
    torch.ops.trb_tde.register_io(PLUGIN)
    srv = _FakeRedis()
    t = threading.Thread(target=srv.serve_forever, daemon=True)
    t.start()
    yield srv
    srv.shutdown()
    srv.server_close()


def _shards(w, m, col_shards):
    shards = torch.classes.trb_tde.LocalShardList()
    step = w.shape[1] // col_shards
    for c in range(col_shards):
        shards.append(0, c * step, w.shape[0], step, [w[:, c * step:(c + 1) * step], m if c == 0 else m.clone()])
    return shards


@pytest.mark.parametrize("col_shards", [1, 2])
def test_evict_then_fetch_through_redis(redis, col_shards):
    rows, dim = 6, 8
    torch.manual_seed(0)
    w, m = torch.randn(rows, dim), torch.randn(rows)
    port = redis.server_address[1]
    ps = torch.classes.trb_tde.PS(f"tbl{col_shards}", _shards(w, m, col_shards), dim, 1, f"redis://127.0.0.1:{port}/?prefix=job7_&db=1&num_threads=2", 2)
    expect_w, expect_m = w[[1, 4, 5]].clone(), m[[1, 4, 5]].clone()
    ps.evict(torch.tensor([[1001, 1], [1004, 4], [1005, 5]], dtype=torch.long))
    with redis.lock:
        keys = [k for k in redis.kv if k.startswith(f"job7_tbl{col_shards}_".encode())]
    assert len(keys) == 3 * 2 * col_shards  # ids x (row, state) x column shards
    assert f"job7_tbl{col_shards}_1004_0_0".encode() in keys
    w.zero_(); m.zero_()
    h = ps.fetch(torch.tensor([[1004, 0], [1001, 2], [1005, 3], [777, 5]], dtype=torch.long), 3, True, -0.5, 0.5)
    h.wait()
    torch.testing.assert_close(w[[2, 0, 3]], expect_w)
    torch.testing.assert_close(m[[2, 0, 3]], expect_m)
    assert w[5].abs().max() <= 0.5 and w[5].abs().sum() > 0  # unknown id: re-initialised
    assert b"MSET" in redis.commands and b"MGET" in redis.commands and b"SELECT" in redis.commands


def test_connection_failure_is_an_error_at_construction(redis):
    w, m = torch.zeros(2, 4), torch.zeros(2)
    with pytest.raises(RuntimeError):
        torch.classes.trb_tde.PS("t", _shards(w, m, 1), 4, 1, "redis://127.0.0.1:1/?timeout_ms=200", 2)
    with pytest.raises((RuntimeError, ValueError)):
        torch.classes.trb_tde.PS("t", _shards(w, m, 1), 4, 1, f"redis://127.0.0.1:{redis.server_address[1]}/?bogus=1", 2)
