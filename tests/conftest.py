import os
import sys

import pytest

ROOT = os.path.abspath(os.path.join(os.path.dirname(__file__), ".."))
PKG_PARENT = os.path.join(ROOT, "amd-pace_b200")
for p in (ROOT, PKG_PARENT):
    if p not in sys.path:
        sys.path.insert(0, p)

GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def golden_dir():
    return GOLDEN


_PAGED_GPU_MODULES = ("test_attn_decode_gpu", "test_attn_mma_gpu", "test_kv_cache_gpu", "test_generator_gpu",
                      "test_llama_gpu", "test_step_graph_gpu")


def pytest_generate_tests(metafunc):
    # the paged GPU tests run twice: 64-token physical pages (the default) and pages of one BMC
    # segment (odd sizes such as 10, 17, 28, 94 tokens), which exercises every chunking mode of the kernels
    if metafunc.module.__name__.split(".")[-1] in _PAGED_GPU_MODULES:
        metafunc.fixturenames.append("kv_page_mode")
        metafunc.parametrize("kv_page_mode", ["page64", "page_tps"], indirect=True)


@pytest.fixture
def kv_page_mode(request, monkeypatch):
    if request.param == "page_tps":
        monkeypatch.setenv("PACE_KV_PAGE_TOKENS", "tps")
    else:
        monkeypatch.delenv("PACE_KV_PAGE_TOKENS", raising=False)
    return request.param
