"""No-op stand-in for the ``nvtx`` package (absent from this image), for running the reference
KV manager's own Python code. Ranges do nothing; the call shapes the reference uses are accepted."""
import contextlib
import functools


class annotate(contextlib.ContextDecorator):
    def __init__(self, message=None, color=None, domain=None, category=None, payload=None):
        self.message = message

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        return False

    def __call__(self, func):
        @functools.wraps(func)
        def inner(*a, **k):
            return func(*a, **k)
        return inner


def start_range(message=None, color=None, domain=None, category=None, payload=None):
    return 0


def end_range(range_id):
    return None


def push_range(message=None, color=None, domain=None, category=None, payload=None):
    return 0


def pop_range(domain=None):
    return None


def mark(message=None, color=None, domain=None, category=None, payload=None):
    return None
