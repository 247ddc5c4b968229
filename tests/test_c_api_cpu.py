"""C API (`libxllm_c.so`): called here through ctypes from the running interpreter, and from a
stand-alone C program that embeds its own interpreter."""
import ctypes
import json
import os
import subprocess
import sys
import sysconfig

import torch

from xllm_b200 import LLM, SamplingParams, _build

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
OPTS = dict(devices="cpu", dtype="float32", block_size=16, num_blocks=64, max_seqs_per_batch=4, max_tokens_per_batch=128,
            enable_graph=False)


def _lib():
    lib = ctypes.CDLL(str(_build.build_c_api()))
    lib.xllm_llm_create.restype = ctypes.c_void_p
    lib.xllm_llm_create.argtypes = [ctypes.c_char_p, ctypes.c_char_p]
    lib.xllm_llm_generate.restype = ctypes.c_void_p
    lib.xllm_llm_generate.argtypes = [ctypes.c_void_p, ctypes.c_char_p, ctypes.c_char_p]
    lib.xllm_llm_stats.restype = ctypes.c_void_p
    lib.xllm_llm_stats.argtypes = [ctypes.c_void_p]
    lib.xllm_free_string.argtypes = [ctypes.c_void_p]
    lib.xllm_llm_destroy.argtypes = [ctypes.c_void_p]
    lib.xllm_last_error.restype = ctypes.c_char_p
    return lib


def test_c_api_through_ctypes_matches_python_api():
    lib = _lib()
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, 32000, (n,), generator=g).tolist() for n in (9, 30)]
    want = [o.outputs[0].token_ids for o in LLM("tiny", **OPTS).generate(
        prompts, SamplingParams(max_tokens=6, temperature=0.0, ignore_eos=True))]
    h = lib.xllm_llm_create(b"tiny", json.dumps(OPTS).encode())
    assert h, lib.xllm_last_error()
    raw = lib.xllm_llm_generate(h, json.dumps(prompts).encode(),
                                json.dumps(dict(max_tokens=6, temperature=0.0, ignore_eos=True)).encode())
    assert raw, lib.xllm_last_error()
    res = json.loads(ctypes.string_at(raw).decode())
    lib.xllm_free_string(raw)
    assert [r["token_ids"] for r in res] == want and res[0]["prompt_tokens"] == 9
    st = lib.xllm_llm_stats(h)
    assert json.loads(ctypes.string_at(st).decode())["steps"] > 0
    lib.xllm_free_string(st)
    lib.xllm_llm_destroy(h)
    assert not lib.xllm_llm_create(b"/no/such/model/dir", b"{}")
    assert b"xllm_llm_create failed" in lib.xllm_last_error()


def test_c_api_from_a_c_program(tmp_path):
    src = tmp_path / "host.c"
    src.write_text(r'''
#include <stdio.h>
#include "xllm.h"
int main(void) {
  xllm_llm* llm = xllm_llm_create("tiny", "{\"devices\": \"cpu\", \"dtype\": \"float32\", \"num_blocks\": 64, \"enable_graph\": false}");
  if (!llm) { printf("create failed: %s\n", xllm_last_error()); return 1; }
  char* out = xllm_llm_generate(llm, "[[1, 2, 3, 4, 5]]", "{\"max_tokens\": 4, \"temperature\": 0.0, \"ignore_eos\": true}");
  if (!out) { printf("generate failed: %s\n", xllm_last_error()); return 2; }
  printf("RESULT %s\n", out);
  xllm_free_string(out);
  xllm_llm_destroy(llm);
  return 0;
}
''')
    lib = _build.build_c_api()
    exe = tmp_path / "host"
    inc = os.path.join(ROOT, "xllm_b200", "csrc", "c_api")
    subprocess.run(["gcc", str(src), "-I", inc, "-o", str(exe), str(lib), f"-Wl,-rpath,{lib.parent}",
                    f"-Wl,-rpath,{sysconfig.get_config_var('LIBDIR')}"], check=True)
    env = dict(os.environ, PYTHONPATH=ROOT + os.pathsep + os.pathsep.join(p for p in sys.path if p))
    r = subprocess.run([str(exe)], env=env, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout + r.stderr
    res = json.loads(r.stdout.split("RESULT ", 1)[1])
    assert len(res[0]["token_ids"]) == 4


def test_cpp_wrapper_from_a_cpp_program(tmp_path):
    """The header-only C++ class over the C API: Initialize / Completions / Call / Sleep / WakeUp."""
    src = tmp_path / "host.cc"
    src.write_text(r'''
#include <iostream>
#include "xllm.hpp"
int main() {
  xllm_b200::LLM llm;
  if (!llm.Initialize("tiny", R"({"devices": "cpu", "dtype": "float32", "num_blocks": 64, "enable_graph": false})")) {
    std::cout << "init failed: " << xllm_b200::LLM::LastError() << "\n";
    return 1;
  }
  const std::string sp = R"({"max_tokens": 4, "temperature": 0.0, "ignore_eos": true})";
  std::string a = llm.Completions("[[1, 2, 3, 4, 5]]", sp);
  llm.Sleep(1);
  llm.WakeUp();
  std::string b = llm.Completions("[[1, 2, 3, 4, 5]]", sp);
  std::string beams = llm.Call("beam_search", R"({"prompt": [1, 2, 3, 4, 5], "beam_width": 2, "max_tokens": 3})");
  std::string rec = llm.Recommend("[[1, 2, 3, 4, 5, 6, 7, 8]]", 3, 2);
  bool threw = false;
  try { llm.Call("no_such_method", "{}"); } catch (const std::exception& e) { threw = true; }
  std::cout << "RESULT " << a << "\nAGAIN " << b << "\nBEAMS " << beams << "\nREC " << rec << "\nTHREW " << threw << "\n";
  return 0;
}
''')
    lib = _build.build_c_api()
    exe = tmp_path / "host_cc"
    inc = os.path.join(ROOT, "xllm_b200", "csrc", "c_api")
    subprocess.run(["g++", "-std=c++17", str(src), "-I", inc, "-o", str(exe), str(lib), f"-Wl,-rpath,{lib.parent}",
                    f"-Wl,-rpath,{sysconfig.get_config_var('LIBDIR')}"], check=True)
    env = dict(os.environ, PYTHONPATH=ROOT + os.pathsep + os.pathsep.join(p for p in sys.path if p))
    r = subprocess.run([str(exe)], env=env, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout + r.stderr
    lines = {l.split(" ", 1)[0]: l.split(" ", 1)[1] for l in r.stdout.splitlines() if " " in l}
    assert json.loads(lines["RESULT"]) == json.loads(lines["AGAIN"]) and len(json.loads(lines["RESULT"])[0]["token_ids"]) == 4
    assert len(json.loads(lines["BEAMS"])) == 2 and lines["THREW"] == "1"
    rec = json.loads(lines["REC"])
    assert len(rec) == 1 and len(rec[0]) == 3 and all(len(it["token_ids"]) == 2 for it in rec[0])
    assert rec[0][0]["logprob"] >= rec[0][1]["logprob"] >= rec[0][2]["logprob"]
