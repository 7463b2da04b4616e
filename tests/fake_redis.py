"""A small in-process Redis stand-in that speaks RESP2 over TCP: enough of the command set for the
registry (PING, AUTH, SELECT, INCR, HSET, HGETALL, PEXPIRE, EXISTS, DEL, SCAN with MATCH/COUNT and real
cursor paging). Test helper only."""
import fnmatch
import socket
import socketserver
import threading
import time


class _Store:
    def __init__(self):
        self.d, self.exp, self.lock = {}, {}, threading.Lock()
        self.commands = []

    def alive(self, k):
        t = self.exp.get(k)
        if t is not None and t <= time.time():
            self.d.pop(k, None)
            self.exp.pop(k, None)
        return k in self.d


def _bulk(b):
    return b"$-1\r\n" if b is None else b"$%d\r\n%s\r\n" % (len(b), b)


def _arr(items):
    return b"*%d\r\n" % len(items) + b"".join(items)


class _Handler(socketserver.StreamRequestHandler):
    def _read_cmd(self):
        line = self.rfile.readline()
        if not line:
            return None
        assert line[:1] == b"*", line
        n = int(line[1:])
        out = []
        for _ in range(n):
            ln = int(self.rfile.readline()[1:])
            out.append(self.rfile.read(ln + 2)[:-2])
        return out

    def handle(self):
        st = self.server.store
        authed = not self.server.password
        while True:
            try:
                cmd = self._read_cmd()
            except (ConnectionError, ValueError):
                return
            if cmd is None:
                return
            name = cmd[0].upper().decode()
            st.commands.append(name)
            if self.server.drop_next:
                self.server.drop_next = False
                self.request.shutdown(socket.SHUT_RDWR)
                return
            if name == "AUTH":
                authed = cmd[-1].decode() == self.server.password
                self.wfile.write(b"+OK\r\n" if authed else b"-WRONGPASS invalid password\r\n")
                continue
            if not authed:
                self.wfile.write(b"-NOAUTH Authentication required.\r\n")
                continue
            with st.lock:
                self.wfile.write(self._run(st, name, cmd[1:]))

    def _run(self, st, name, a):
        if name == "PING":
            return b"+PONG\r\n"
        if name == "SELECT":
            return b"+OK\r\n"
        if name == "INCR":
            k = a[0]
            v = int(st.d.get(k, b"0")) + 1
            st.d[k] = str(v).encode()
            return b":%d\r\n" % v
        if name == "HSET":
            k = a[0]
            st.alive(k)
            h = st.d.setdefault(k, {})
            new = 0
            for i in range(1, len(a), 2):
                new += a[i] not in h
                h[a[i]] = a[i + 1]
            return b":%d\r\n" % new
        if name == "HGETALL":
            h = st.d.get(a[0], {}) if st.alive(a[0]) else {}
            flat = []
            for f, v in h.items():
                flat += [_bulk(f), _bulk(v)]
            return _arr(flat)
        if name == "PEXPIRE":
            if not st.alive(a[0]):
                return b":0\r\n"
            st.exp[a[0]] = time.time() + int(a[1]) / 1000.0
            return b":1\r\n"
        if name == "EXISTS":
            return b":%d\r\n" % sum(st.alive(k) for k in a)
        if name == "DEL":
            n = 0
            for k in a:
                n += st.d.pop(k, None) is not None
                st.exp.pop(k, None)
            return b":%d\r\n" % n
        if name == "SCAN":
            cursor = int(a[0])
            pat, count = b"*", 10
            for i in range(1, len(a) - 1, 2):
                if a[i].upper() == b"MATCH":
                    pat = a[i + 1]
                if a[i].upper() == b"COUNT":
                    count = int(a[i + 1])
            count = min(count, self.server.scan_page)
            keys = sorted(k for k in list(st.d) if st.alive(k))
            page = keys[cursor:cursor + count]
            nxt = cursor + count if cursor + count < len(keys) else 0
            hit = [_bulk(k) for k in page if fnmatch.fnmatchcase(k.decode(), pat.decode())]
            return _arr([_bulk(str(nxt).encode()), _arr(hit)])
        return b"-ERR unknown command '%s'\r\n" % name.encode()


class FakeRedis(socketserver.ThreadingTCPServer):
    allow_reuse_address = True
    daemon_threads = True

    def __init__(self, password: str = "", scan_page: int = 7):
        super().__init__(("127.0.0.1", 0), _Handler)
        self.store, self.password, self.scan_page, self.drop_next = _Store(), password, scan_page, False
        self.port = self.server_address[1]
        self._th = threading.Thread(target=self.serve_forever, daemon=True)
        self._th.start()

    def stop(self):
        self.shutdown()
        self.server_close()
