"""Import-only stand-in for ``redis`` (absent from this image). The reference imports it at module
load in its distributed-index wrapper; the single-node paths this repository's reference arm runs
never open a connection, so constructing a client raises."""


class RedisError(Exception):
    pass


class ConnectionError(RedisError):
    pass


class TimeoutError(RedisError):
    pass


class Redis:
    def __init__(self, *a, **k):
        raise ConnectionError("redis is not available on this image")

    @classmethod
    def from_url(cls, *a, **k):
        raise ConnectionError("redis is not available on this image")


StrictRedis = Redis


class _Exceptions:
    RedisError = RedisError
    ConnectionError = ConnectionError
    TimeoutError = TimeoutError


exceptions = _Exceptions
