from .swa_host_pool import SWAHostPool

__all__ = ["SWAHostPool"]
