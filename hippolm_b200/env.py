"""Process environment set-up done before the heavy imports (``src/training/env.py:45-241``).

* ``.env`` loader (KEY=VALUE lines; existing variables win)
* NCCL pinning for one NVSwitch node: P2P over NVLink, no InfiniBand, loopback rendezvous.
  The reference disables the NCCL watchdog because first-step Triton compilation stalls the
  heartbeat for minutes; nothing is JIT-compiled here, so the watchdog stays on with a normal timeout.
* cache-directory routing (``HIPPOLM_CACHE_DIR``, HF / ModelScope caches under the repo)
"""
from __future__ import annotations

import os
from typing import Dict, Optional

_NCCL_DEFAULTS = {
    "NCCL_P2P_LEVEL": "NVL",
    "NCCL_IB_DISABLE": "1",
    "NCCL_SOCKET_IFNAME": "^docker,veth,br-",
    "TORCH_NCCL_ASYNC_ERROR_HANDLING": "1",
    "TORCH_NCCL_HEARTBEAT_TIMEOUT_SEC": "600",
    "CUDA_DEVICE_MAX_CONNECTIONS": "8",
}


def load_dotenv(path: str = ".env", env: Optional[Dict[str, str]] = None) -> Dict[str, str]:
    env = os.environ if env is None else env
    loaded: Dict[str, str] = {}
    if not os.path.exists(path):
        return loaded
    with open(path) as f:
        for line in f:
            line = line.strip()
            if not line or line.startswith("#") or "=" not in line:
                continue
            k, v = line.split("=", 1)
            k, v = k.strip(), v.strip().strip('"').strip("'")
            if k and k not in env:
                env[k] = v
                loaded[k] = v
    return loaded


def pin_nccl_environment(env: Optional[Dict[str, str]] = None) -> None:
    env = os.environ if env is None else env
    for k, v in _NCCL_DEFAULTS.items():
        env.setdefault(k, v)


def get_cache_dir(env: Optional[Dict[str, str]] = None) -> str:
    env = os.environ if env is None else env
    d = env.get("HIPPOLM_CACHE_DIR")
    if not d:
        d = os.path.join(os.getcwd(), ".cache", "hippolm", "datasets")
    return d


def pin_cache_directories(repo_root: Optional[str] = None, env: Optional[Dict[str, str]] = None) -> None:
    env = os.environ if env is None else env
    root = repo_root or os.getcwd()
    env.setdefault("MODELSCOPE_CACHE", os.path.join(root, ".cache", "modelscope"))
    env.setdefault("HF_HOME", os.path.join(root, ".cache", "huggingface"))
    env.setdefault("HF_DATASETS_CACHE", os.path.join(env["HF_HOME"], "datasets"))


def configure_runtime_environment(cache_dir: Optional[str] = None, dotenv: str = ".env") -> None:
    load_dotenv(dotenv)
    if cache_dir:
        os.environ["HIPPOLM_CACHE_DIR"] = cache_dir
    os.environ.setdefault("HF_ENDPOINT", "https://huggingface.co")
    os.environ.setdefault("HF_DATASETS_DOWNLOAD_RETRIES", "5")
    pin_nccl_environment()
    pin_cache_directories()
    import socket
    socket.setdefaulttimeout(60.0)
