"""View of a TensorRT-LLM ``LlmRequest`` with the fields the connector reads
(flexkv/integration/tensorrt_llm/utils.py:14-74). Duck-typed: anything with the same
attributes works, so the adapter is testable without TensorRT-LLM installed."""
from __future__ import annotations

from typing import Any, List, Optional

import numpy as np


class RequestWrapper:
    def __init__(self, request: Any) -> None:
        self._request = request
        self._np_tokens: Optional[np.ndarray] = None

    @property
    def req_id(self):
        rid = getattr(self._request, "request_id", None)
        return rid if rid is not None else getattr(self._request, "py_request_id", None)

    request_id = req_id

    @property
    def all_token_ids(self) -> List[int]:
        r = self._request
        if hasattr(r, "get_tokens"):
            try:
                toks = r.get_tokens()
            except TypeError:                       # bindings that want the beam index
                return list(r.get_tokens(0))
            if len(toks) and isinstance(toks[0], (list, tuple, np.ndarray)):
                if len(toks) != 1:
                    raise ValueError("beam search is not supported: the cache holds one sequence per request")
                return list(toks[0])
            return list(toks)
        return list(getattr(r, "tokens", []))

    @property
    def np_token_ids(self) -> np.ndarray:
        """The list -> numpy conversion is cached: match and put read the tokens several times per step."""
        if self._np_tokens is None or len(self._np_tokens) != self.num_tokens:
            self._np_tokens = np.asarray(self.all_token_ids, dtype=np.int64)
        return self._np_tokens

    @property
    def num_tokens(self) -> int:
        return len(self.all_token_ids)

    @property
    def num_prompt_tokens(self) -> int:
        return int(getattr(self._request, "prompt_len", self.num_tokens))

    @property
    def num_new_matched_tokens(self) -> int:
        return int(getattr(self._request, "num_connector_matched_tokens", 0) or 0)

    def _flag(self, name: str, default: bool = True) -> bool:
        v = getattr(self._request, name, default)
        return bool(v() if callable(v) else v)

    def is_finished(self) -> bool:
        return self._flag("is_finished")

    def is_finished_normal(self) -> bool:
        return self._flag("is_finished_normal")

    # ---- what the scheduler core reads off a request -------------------------------------------------
    lora_request = None

    @property
    def namespace_info(self) -> Optional[List[str]]:
        return extract_namespace(self._request)

    @property
    def cache_salt(self):
        return None          # folded into namespace_info, in the reference's order

    def __repr__(self) -> str:
        return (f"RequestWrapper(req_id={self.req_id}, num_prompt_tokens={self.num_prompt_tokens}, "
                f"num_tokens={self.num_tokens}, num_new_matched_tokens={self.num_new_matched_tokens})")


def extract_namespace(request: Any) -> Optional[List[str]]:
    """Cache-isolation namespace of a request, most significant component first: the LoRA task id, the
    cache salt id, then the user's ``namespace_info`` (a string whose ``|``-separated parts form a
    hierarchy, e.g. ``"tenant_A|user_1"``). None when the request carries none of them
    (flexkv/integration/tensorrt_llm/trtllm_adapter.py:102-151)."""
    ns: List[str] = []
    lora = getattr(request, "lora_task_id", None)
    if lora is not None:
        ns.append(str(lora))
    salt = getattr(request, "cache_salt_id", None)
    if salt is not None:
        ns.append(str(salt))
    user = getattr(request, "namespace_info", None)
    if user is not None:
        if isinstance(user, str):
            ns.extend(part.strip() for part in user.split("|") if part.strip())
        elif isinstance(user, (list, tuple)):
            ns.extend(str(part) for part in user)
        else:
            ns.append(str(user))
    return ns or None


def physical_device_id(logical: int, visible: Optional[str]) -> int:
    """CUDA_VISIBLE_DEVICES renumbers devices per process; the data plane, which lives in another process,
    needs the physical index (flexkv/integration/tensorrt_llm/trtllm_adapter.py:551-563)."""
    if not visible:
        return logical
    try:
        ids = [int(x) for x in visible.split(",") if x.strip() != ""]
    except ValueError:
        return logical          # UUID-style lists cannot be mapped here
    return ids[logical] if 0 <= logical < len(ids) else logical
