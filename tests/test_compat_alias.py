"""The ``flexkv`` import alias (``compat/``) and the method surface that vLLM's built-in connector shim calls."""
import ast
import importlib.util
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_reference_module_paths_resolve_to_the_same_objects():
    code = (
        "import flexkv, flexkv_b200\n"
        "from flexkv.integration.vllm.vllm_v1_adapter import FlexKVConnectorV1Impl as A\n"
        "from flexkv_b200.integration.vllm.vllm_v1_adapter import FlexKVConnectorV1Impl as B\n"
        "from flexkv.kvmanager import KVManager as KA\n"
        "from flexkv.common.config import CacheConfig as CA\n"
        "import flexkv.integration.sglang.connector as S, flexkv_b200.integration.sglang.connector as S2\n"
        "from flexkv.integration.tensorrt_llm.trtllm_adapter import FlexKVSchedulerConnector, FlexKVWorkerConnector\n"
        "from flexkv.server.client import KVTPClient, KVDPClient\n"
        "import sys\n"
        "assert A is B and KA is flexkv_b200.KVManager and CA is flexkv_b200.CacheConfig and S is S2\n"
        "assert flexkv is flexkv_b200 and sys.modules['flexkv.kvmanager'] is sys.modules['flexkv_b200.kvmanager']\n"
        "try:\n"
        "    import flexkv.no_such_module\n"
        "    raise SystemExit('missing modules must stay missing')\n"
        "except ImportError:\n"
        "    pass\n"
        "print('alias ok')\n")
    env = dict(os.environ, PYTHONPATH=os.pathsep.join([os.path.join(ROOT, "compat"), ROOT]))
    p = subprocess.run([sys.executable, "-c", code], env=env, capture_output=True, text=True, timeout=120)
    assert p.returncode == 0 and "alias ok" in p.stdout, p.stdout + p.stderr


def test_every_call_of_vllms_connector_shim_exists_here():
    """vLLM ships ``FlexKVConnectorV1``, which forwards to ``FlexKVConnectorV1Impl``: every method it calls on
    the implementation object must exist on this package's class (read from vLLM's source, nothing imported)."""
    spec = importlib.util.find_spec("vllm")
    if spec is None or not spec.submodule_search_locations:
        pytest.skip("vllm is not installed")
    path = os.path.join(list(spec.submodule_search_locations)[0], "distributed", "kv_transfer", "kv_connector", "v1",
                        "flexkv_connector.py")
    if not os.path.exists(path):
        pytest.skip("this vllm has no built-in FlexKV connector shim")
    tree = ast.parse(open(path).read())
    called = set()
    for node in ast.walk(tree):
        if isinstance(node, ast.Call) and isinstance(node.func, ast.Attribute):
            v = node.func.value
            if isinstance(v, ast.Attribute) and v.attr == "_flexkv_connector":
                called.add(node.func.attr)
    assert called, "the shim's forwarding calls were not found"
    from flexkv_b200.integration.vllm.vllm_v1_adapter import FlexKVConnectorV1Impl
    missing = sorted(m for m in called if not callable(getattr(FlexKVConnectorV1Impl, m, None)))
    assert not missing, f"vLLM's shim calls methods this implementation lacks: {missing}"


def test_connector_returns_vllms_own_types_when_vllm_is_there():
    """vLLM's scheduler output carries a ``KVConnectorMetadata`` and its logger aggregates ``KVConnectorStats``;
    what the implementation returns must be instances of those (checked in a child process: importing vLLM
    takes a while and configures logging)."""
    if importlib.util.find_spec("vllm") is None:
        pytest.skip("vllm is not installed")
    code = (
        "import pickle\n"
        "from vllm.distributed.kv_transfer.kv_connector.v1.base import KVConnectorMetadata\n"
        "from vllm.distributed.kv_transfer.kv_connector.v1.metrics import KVConnectorStats\n"
        "from flexkv_b200.integration.vllm.vllm_v1_adapter import _vllm_types\n"
        "t = _vllm_types()\n"
        "m = t['meta']({'a'}, {'b', 'c'})\n"
        "assert isinstance(m, KVConnectorMetadata) and m['finished_recving'] == {'b', 'c'}\n"
        "s = t['stats'](data=dict(num_get_query_tokens=100, num_gpu_matched_tokens=25, num_flexkv_matched_tokens=50))\n"
        "assert isinstance(s, KVConnectorStats) and not s.is_empty()\n"
        "s2 = pickle.loads(pickle.dumps(s))\n"
        "s.aggregate(s2)\n"
        "r = s.reduce()\n"
        "assert r['num_get_query_tokens'] == 200 and abs(r['get_flexkv_match_ratio'] - 0.5) < 1e-9, r\n"
        "s.reset(); assert s.data == {}\n"
        "print('types ok')\n")
    env = dict(os.environ, PYTHONPATH=ROOT)
    p = subprocess.run([sys.executable, "-c", code], env=env, capture_output=True, text=True, timeout=300, cwd="/tmp")
    assert p.returncode == 0 and "types ok" in p.stdout, (p.stdout + p.stderr)[-3000:]
