"""Builds the small native helpers the tests use (in-tree, on demand)."""
import os
import subprocess

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CPP = os.path.join(ROOT, "tests", "cpp")
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
API_TESTS_SO = os.path.join(CPP, "libcusync_api_tests.so")
POLICY_EVAL_SO = os.path.join(CPP, "libcusync_policy_eval_host.so")


def _stale(target, sources):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(s) > t for s in sources)


def _headers():
    out = []
    for root, _, files in os.walk(os.path.join(ROOT, "include")):
        out += [os.path.join(root, f) for f in files]
    return out


def build_library():
    from cusync_b200 import build as b
    return b.build()


def build_api_tests():
    lib = build_library()
    src = os.path.join(CPP, "api_tests.cu")
    if _stale(API_TESTS_SO, [src, lib] + _headers()):
        subprocess.check_call(
            [NVCC, "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O2", "-std=c++17", "-shared",
             "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden", "-I", os.path.join(ROOT, "include"), src,
             "-o", API_TESTS_SO, "-L", os.path.join(ROOT, "cusync_b200"), "-lcusync_b200",
             "-Xlinker", "-rpath", "-Xlinker", "$ORIGIN/../../cusync_b200"],
            stderr=subprocess.DEVNULL)
    return API_TESTS_SO


def build_policy_eval_host():
    src = os.path.join(CPP, "policy_eval_host.cpp")
    if _stale(POLICY_EVAL_SO, [src] + _headers()):
        subprocess.check_call(["/usr/bin/g++", "-O2", "-std=c++17", "-shared", "-fPIC", "-fvisibility=hidden",
                               "-I", os.path.join(ROOT, "include"), src, "-o", POLICY_EVAL_SO])
    return POLICY_EVAL_SO


def build_all():
    build_library()
    build_api_tests()
    build_policy_eval_host()
