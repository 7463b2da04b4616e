"""In-box registry: node ids, liveness, node metadata and the block-record store that
the cross-node index publishes into.

The reference keeps this state in Redis (flexkv/cache/redis_meta.py:158-906,
csrc/dist/redis_meta_channel.cpp:198-215). The same roles and the same key schema are
served here by a small store that lives inside the box:

* ``global:node_id``                    counter, allocates node ids (INCR);
* ``node:<id>``                         hash {node_id, ip, uuid, status, timestamp, pp_rank, pp_size} with a TTL that
                                        a heartbeat thread renews; an expired key is never resurrected — the node
                                        must register again and gets a new id;
* ``meta:<id>[:pp<rank>]``              hash with what a peer needs to read this node's host pool
                                        (pool file, block bytes, block count, zmq address);
* ``<CPUB|SSDB>:block:<nid>:<hash-hex>`` hash {ph, pb, nid, hash, lt, state}, one per published block.

``RegistryStore`` is the data structure, ``RegistryServer`` serves it over a ZeroMQ REP
socket so that several processes of one box (or several boxes) share it, and
``RegistryClient`` talks either to a server endpoint or straight to a store object living
in the same process. ``redis_client.RedisRegistryClient`` has the same methods over the Redis wire
protocol (``connect("redis://host", port)``), so the registry can also live in a Redis server.
"""
from __future__ import annotations

import pickle
import threading
import time
import uuid as _uuid
from typing import Any, Callable, Dict, Iterable, List, Optional, Sequence, Tuple

from ..common.debug import flexkv_logger


class RegistryStore:
    """Hash-valued keys with optional expiry, counters, prefix scans."""

    def __init__(self, clock: Callable[[], float] = time.time) -> None:
        self._d: Dict[str, Dict[str, Any]] = {}
        self._exp: Dict[str, float] = {}
        self._ctr: Dict[str, int] = {}
        self._lock = threading.Lock()
        self._clock = clock

    def _alive(self, key: str) -> bool:
        t = self._exp.get(key)
        if t is not None and t <= self._clock():
            self._d.pop(key, None)
            self._exp.pop(key, None)
            return False
        return key in self._d

    # every public method is one atomic command
    def incr(self, key: str) -> int:
        with self._lock:
            self._ctr[key] = self._ctr.get(key, 0) + 1
            return self._ctr[key]

    def hset(self, key: str, mapping: Dict[str, Any], ttl: Optional[float] = None, only_if_exists: bool = False) -> bool:
        with self._lock:
            alive = self._alive(key)
            if only_if_exists and not alive:
                return False
            self._d.setdefault(key, {}).update(mapping)
            if ttl is not None:
                self._exp[key] = self._clock() + ttl
            return True

    def hset_many(self, items: Sequence[Tuple[str, Dict[str, Any]]]) -> int:
        with self._lock:
            for key, mapping in items:
                self._alive(key)
                self._d.setdefault(key, {}).update(mapping)
            return len(items)

    def hgetall(self, key: str) -> Dict[str, Any]:
        with self._lock:
            return dict(self._d[key]) if self._alive(key) else {}

    def expire(self, key: str, ttl: float) -> bool:
        """Renews a TTL; False when the key is already gone (no resurrection)."""
        with self._lock:
            if not self._alive(key):
                return False
            self._exp[key] = self._clock() + ttl
            return True

    def exists(self, key: str) -> bool:
        with self._lock:
            return self._alive(key)

    def delete(self, keys: Iterable[str]) -> int:
        n = 0
        with self._lock:
            for k in keys:
                n += int(self._d.pop(k, None) is not None)
                self._exp.pop(k, None)
        return n

    def scan(self, prefix: str) -> List[str]:
        with self._lock:
            return sorted(k for k in list(self._d) if k.startswith(prefix) and self._alive(k))

    def scan_values(self, prefix: str) -> List[Dict[str, Any]]:
        with self._lock:
            return [dict(self._d[k]) for k in list(self._d) if k.startswith(prefix) and self._alive(k)]

    def delete_prefix(self, prefix: str) -> int:
        with self._lock:
            ks = [k for k in self._d if k.startswith(prefix)]
            for k in ks:
                self._d.pop(k, None)
                self._exp.pop(k, None)
            return len(ks)


_COMMANDS = ("incr", "hset", "hset_many", "hgetall", "expire", "exists", "delete", "scan", "scan_values",
             "delete_prefix")

_INPROC: Dict[str, RegistryStore] = {}
_INPROC_LOCK = threading.Lock()


def inproc_store(name: str) -> RegistryStore:
    """Process-wide named store (several managers in one process share it)."""
    with _INPROC_LOCK:
        if name not in _INPROC:
            _INPROC[name] = RegistryStore()
        return _INPROC[name]


class RegistryServer:
    """Serves a store on a ZeroMQ REP socket (``tcp://127.0.0.1:port`` or ``ipc://path``)."""

    def __init__(self, endpoint: str, store: Optional[RegistryStore] = None) -> None:
        import zmq
        self.store = store or RegistryStore()
        self.endpoint = endpoint
        self._ctx = zmq.Context.instance()
        self._sock = self._ctx.socket(zmq.REP)
        self._sock.setsockopt(zmq.LINGER, 0)
        self._sock.bind(endpoint)
        self._stop = threading.Event()
        self._th = threading.Thread(target=self._loop, name="flexkv-registry", daemon=True)
        self._th.start()

    def _loop(self) -> None:
        import zmq
        poller = zmq.Poller()
        poller.register(self._sock, zmq.POLLIN)
        while not self._stop.is_set():
            if not dict(poller.poll(100)):
                continue
            try:
                cmd, args, kwargs = pickle.loads(self._sock.recv())
                if cmd not in _COMMANDS:
                    raise ValueError(f"unknown registry command {cmd!r}")
                reply = (True, getattr(self.store, cmd)(*args, **kwargs))
            except Exception as e:  # noqa: BLE001
                reply = (False, repr(e))
            self._sock.send(pickle.dumps(reply))

    def close(self) -> None:
        self._stop.set()
        self._th.join(timeout=2)
        self._sock.close()


class RegistryClient:
    """``target`` is a RegistryStore (same process) or a server endpoint string."""

    def __init__(self, target, timeout_ms: int = 3000) -> None:
        self._store = target if isinstance(target, RegistryStore) else None
        self._endpoint = None if self._store is not None else str(target)
        self._timeout_ms = timeout_ms
        self._local = threading.local()

    def _sock(self):
        import zmq
        s = getattr(self._local, "sock", None)
        if s is None:
            s = zmq.Context.instance().socket(zmq.REQ)
            s.setsockopt(zmq.LINGER, 0)
            s.setsockopt(zmq.RCVTIMEO, self._timeout_ms)
            s.setsockopt(zmq.SNDTIMEO, self._timeout_ms)
            s.connect(self._endpoint)
            self._local.sock = s
        return s

    def _call(self, cmd: str, *args, **kwargs):
        if self._store is not None:
            return getattr(self._store, cmd)(*args, **kwargs)
        import zmq
        s = self._sock()
        try:
            s.send(pickle.dumps((cmd, args, kwargs)))
            ok, val = pickle.loads(s.recv())
        except zmq.ZMQError as e:
            # a REQ socket that missed its reply cannot be reused
            s.close()
            self._local.sock = None
            raise ConnectionError(f"registry at {self._endpoint} did not answer: {e}") from e
        if not ok:
            raise RuntimeError(f"registry command {cmd} failed: {val}")
        return val

    def __getattr__(self, name: str):
        if name in _COMMANDS:
            return lambda *a, **k: self._call(name, *a, **k)
        raise AttributeError(name)


def connect(host: str, port: int, password: Optional[str] = None) -> RegistryClient:
    """``host`` "inproc[:name]" selects a store inside this process; anything else is the
    address of a RegistryServer (the configuration reuses the reference's redis_host/redis_port fields);
    "redis://[:password@]host[:port][/db]" is a Redis server."""
    if host.startswith("inproc"):
        name = host.split(":", 1)[1] if ":" in host else "default"
        return RegistryClient(inproc_store(name))
    if host.startswith("redis://"):
        # a Redis server, spoken to over its wire protocol: redis://[:password@]host[/db]
        from .redis_client import RedisRegistryClient
        rest = host[len("redis://"):]
        password, db = password or "", 0
        if "@" in rest:
            cred, rest = rest.rsplit("@", 1)
            password = cred.split(":", 1)[1] if ":" in cred else cred
        if "/" in rest:
            rest, dbs = rest.split("/", 1)
            db = int(dbs or 0)
        if ":" in rest:
            rest, ps = rest.rsplit(":", 1)
            port = int(ps)
        return RedisRegistryClient(rest, port or 6379, password=password, db=db)
    if host.startswith("ipc://") or host.startswith("tcp://"):
        return RegistryClient(host)
    return RegistryClient(f"tcp://{host}:{port}")


class NodeRegistry:
    """Node id allocation, heartbeat and node metadata (reference: RedisMeta,
    flexkv/cache/redis_meta.py:296-430,514-617,796-846)."""

    def __init__(self, client: RegistryClient, ip: str = "127.0.0.1", pp_rank: int = 0, pp_size: int = 1,
                 node_ttl_seconds: float = 10.0, heartbeat_interval: Optional[float] = None,
                 instance_uuid: Optional[str] = None) -> None:
        self.client = client
        self.ip, self.pp_rank, self.pp_size = ip, pp_rank, pp_size
        self.ttl = float(node_ttl_seconds)
        self.interval = heartbeat_interval if heartbeat_interval is not None else max(0.05, self.ttl / 3)
        self.uuid = instance_uuid or _uuid.uuid4().hex
        self.node_id: Optional[int] = None
        self.lost = threading.Event()      # set when the heartbeat found the node key expired
        self._stop = threading.Event()
        self._th: Optional[threading.Thread] = None

    # ---- registration -------------------------------------------------------------
    def register(self, cleanup_stale: bool = True) -> int:
        if cleanup_stale:
            self.cleanup_same_identity()
        nid = int(self.client.incr("global:node_id"))
        self.client.hset(f"node:{nid}", dict(node_id=nid, ip=self.ip, uuid=self.uuid, status="active",
                                             timestamp=time.time(), pp_rank=self.pp_rank, pp_size=self.pp_size),
                         ttl=self.ttl)
        self.node_id = nid
        self.lost.clear()
        return nid

    def cleanup_same_identity(self) -> int:
        """Removes records of earlier incarnations of this instance (same ip and uuid)."""
        n = 0
        for rec in self.client.scan_values("node:"):
            if rec.get("ip") == self.ip and rec.get("uuid") == self.uuid:
                n += 1
                self.remove_node(int(rec["node_id"]))
        return n

    def remove_node(self, nid: int) -> None:
        self.client.delete([f"node:{nid}"])
        self.client.delete_prefix(f"meta:{nid}")
        for kind in ("CPUB", "SSDB", "PCFSB"):
            self.client.delete_prefix(f"{kind}:block:{nid}:")

    def start_heartbeat(self) -> None:
        if self._th is not None:
            return
        self._stop.clear()
        self._th = threading.Thread(target=self._beat, name="flexkv-node-heartbeat", daemon=True)
        self._th.start()

    def _beat(self) -> None:
        while not self._stop.wait(self.interval):
            try:
                if not self.client.expire(f"node:{self.node_id}", self.ttl):
                    flexkv_logger.error("node %s expired in the registry; it must register again", self.node_id)
                    self.lost.set()
                    return
                for k in self.client.scan(f"meta:{self.node_id}"):
                    self.client.expire(k, self.ttl)
            except (ConnectionError, RuntimeError) as e:
                flexkv_logger.warning("registry heartbeat failed: %s", e)

    def stop(self, unregister: bool = True) -> None:
        self._stop.set()
        if self._th is not None:
            self._th.join(timeout=2)
            self._th = None
        if unregister and self.node_id is not None:
            try:
                self.remove_node(self.node_id)
            except (ConnectionError, RuntimeError):
                pass

    # ---- queries ---------------------------------------------------------------------
    def active_nodes(self) -> List[int]:
        return sorted(int(r["node_id"]) for r in self.client.scan_values("node:") if r.get("status") == "active")

    def set_node_meta(self, meta: Dict[str, Any]) -> None:
        key = f"meta:{self.node_id}" + (f":pp{self.pp_rank}" if self.pp_size > 1 else "")
        self.client.hset(key, dict(meta, pp_rank=self.pp_rank, pp_size=self.pp_size), ttl=self.ttl)

    def get_node_meta(self, nid: int, pp_rank: Optional[int] = None) -> Dict[str, Any]:
        if pp_rank is not None:
            m = self.client.hgetall(f"meta:{nid}:pp{pp_rank}")
            if m:
                return m
        return self.client.hgetall(f"meta:{nid}")

    # ---- reset barrier -----------------------------------------------------------------
    def reset_barrier(self, epoch: int, timeout: float = 10.0, poll: float = 0.01) -> bool:
        """Every live node acknowledges reset ``epoch``; returns once all of them did
        (reference: flexkv/cache/hie_cache_engine.py:177-223)."""
        self.client.hset(f"reset:{epoch}", {str(self.node_id): 1}, ttl=max(timeout * 2, 5.0))
        deadline = time.time() + timeout
        while time.time() < deadline:
            acks = self.client.hgetall(f"reset:{epoch}")
            if all(str(n) in acks for n in self.active_nodes()):
                return True
            time.sleep(max(0.001, poll))
        return False


class RegistryMetaChannel:
    """Block records of the cross-node index in the registry. The method set is the
    native MetaChannel interface (rows are (ph, pb, nid, hash, lt, state) tuples); only
    nodes whose ``node:<id>`` key is alive are listed, so a dead node's blocks drop out
    of every peer's view once its TTL runs out."""

    def __init__(self, client: RegistryClient, kind: str = "CPUB") -> None:
        self.client, self.kind = client, kind

    def _key(self, nid: int, h: int) -> str:
        return f"{self.kind}:block:{int(nid)}:{int(h) & 0xFFFFFFFFFFFFFFFF:016x}"

    def publish(self, nid: int, rows) -> None:
        self.client.hset_many([(self._key(nid, r[3]), dict(ph=int(r[0]), pb=int(r[1]), nid=int(r[2]), hash=int(r[3]),
                                                           lt=int(r[4]), state=int(r[5]))) for r in rows])

    def remove(self, nid: int, hashes) -> None:
        self.client.delete([self._key(nid, h) for h in hashes])

    def list_nodes(self) -> List[int]:
        return sorted(int(r["node_id"]) for r in self.client.scan_values("node:") if r.get("status") == "active")

    def load(self, nid: int):
        return [(r["ph"], r["pb"], r["nid"], r["hash"], r["lt"], r["state"])
                for r in self.client.scan_values(f"{self.kind}:block:{int(nid)}:")]

    def clear_node(self, nid: int) -> None:
        self.client.delete_prefix(f"{self.kind}:block:{int(nid)}:")
