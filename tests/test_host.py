"""CPU tests of the host side: the C-ABI library loads and exports every declared symbol,
config / model-file parsing and error codes, sharding logic under gloo."""
import ctypes as C
import os
import re

import numpy as np
import pytest

from linmt_b200 import modelfile, synth

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_exports_every_declared_symbol(cuda_lib):
    hdr = open(os.path.join(ROOT, "include", "linmt_decoder.h")).read()
    hdr = re.sub(r"/\*.*?\*/", "", hdr, flags=re.S)
    names = set(re.findall(r"\b((?:linmt|python)_[a-z_0-9]+)\s*\(", hdr))
    assert {"python_decoder_init", "python_decoder_do_job", "linmt_decode_batch", "linmt_create"} <= names
    for n in names:
        assert hasattr(cuda_lib, n), f"{n} is declared in include/linmt_decoder.h but not exported"


def test_blob_floats_matches_generator(cuda_lib):
    from linmt_b200 import _lib
    for d in (synth.ModelDesc(2, 128, 1000, 1000, 1), synth.ModelDesc(4, 1000, 30000, 30000, 1),
              synth.ModelDesc(3, 64, 200, 100, 0)):
        dc = _lib.ModelDescC(d.L, d.H, d.V, d.Vs, d.feed_input)
        assert cuda_lib.linmt_blob_floats(C.byref(dc)) == synth.blob_floats(d)


def test_default_options_are_the_reference_defaults(cuda_lib):
    from linmt_b200 import _lib
    o = _lib.OptionsC()
    cuda_lib.linmt_default_options(C.byref(o))
    # src/global_configuration.h:228-235
    assert (o.beam, o.nbest) == (12, 1)
    assert abs(o.lp_alpha - 0.65) < 1e-7 and abs(o.cp_beta - 0.2) < 1e-7
    assert (o.min_ratio, o.max_ratio, o.penalty, o.diversity) == (0.5, 1.5, 0.0, 0.0)
    assert o.attention_d == 10


def test_create_errors_without_touching_the_gpu(cuda_lib, tmp_path):
    h = C.c_void_p()
    assert cuda_lib.linmt_create(str(tmp_path / "missing.config").encode(), C.byref(h)) == 3  # LINMT_EIO
    cfg = tmp_path / "a.config"
    cfg.write_text('# comment\nparam="--beam-size" value="4"\n')
    assert cuda_lib.linmt_create(str(cfg).encode(), C.byref(h)) == 1  # missing --nmt-model
    assert b"--nmt-model" in cuda_lib.linmt_front_error()
    cfg.write_text('param="--nmt-model" value="/nonexistent/model"\nparam="--beam-size" value="0"\n')
    assert cuda_lib.linmt_create(str(cfg).encode(), C.byref(h)) == 1
    assert b"beam-size" in cuda_lib.linmt_front_error()
    cfg.write_text('param="--nmt-model" value="/nonexistent/model"\nparam="--decoding-ratio" value="2 1"\n')
    assert cuda_lib.linmt_create(str(cfg).encode(), C.byref(h)) == 1
    cfg.write_text('param="--nmt-model" value="/nonexistent/model"\n')
    assert cuda_lib.linmt_create(str(cfg).encode(), C.byref(h)) == 3
    # a truncated model file is an I/O error, never a crash
    d = synth.ModelDesc(1, 8, 20, 10, 1)
    blob = synth.make_blob(d, 0)
    mp = tmp_path / "m.txt"
    modelfile.write_model(str(mp), d, blob)
    data = mp.read_bytes()
    mp.write_bytes(data[: len(data) // 2])
    cfg.write_text(f'param="--nmt-model" value="{mp}"\n')
    assert cuda_lib.linmt_create(str(cfg).encode(), C.byref(h)) == 3
    assert b"truncated" in cuda_lib.linmt_front_error() or b"bad number" in cuda_lib.linmt_front_error()


def test_do_job_before_init_returns_empty(cuda_lib):
    assert cuda_lib.python_decoder_do_job(b"hello world") == b""
    assert cuda_lib.python_decoder_do_job(b"") == b""


def test_model_file_roundtrip_text_and_binary(tmp_path):
    """The writer's text form parses back to the same floats (checked through numpy here; the
    C++ reader is exercised on the GPU tests)."""
    d = synth.ModelDesc(1, 4, 6, 5, 1)
    blob = synth.make_blob(d, 3)
    p = tmp_path / "m.txt"
    modelfile.write_model(str(p), d, blob)
    lines = p.read_text().split("\n")
    assert lines[0].split() == ["1", "4", "6", "5", "1", "1", "0", "0", "0"]
    body = lines[1 + 1 + 5 + 1 + 6 + 1:]
    vals = []
    off = 0
    i = 0
    for _, r, c in synth.blob_layout(d):
        m = np.array([[float(x) for x in body[i + rr].split()] for rr in range(r)], np.float32)
        assert m.shape == (r, c)
        assert body[i + r] == ""
        np.testing.assert_array_equal(m.T.reshape(-1), blob[off:off + r * c])
        i += r + 1
        off += r * c


def _shard_worker(rank, world, port, q):
    import torch.distributed as dist
    from linmt_b200 import shard
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    c = synth.configs()["C1"]
    sents = c.sentences(23)
    mine = shard.partition(sents, world, batch=4)[rank]
    # stand-in decode: a deterministic function of the sentence (sum of ids, length)
    local = {int(i): (int(sents.ids[sents.off[i]:sents.off[i + 1]].sum()), int(sents.steps[i])) for i in mine}
    merged = shard.gather_results(local, dst=0)
    if rank == 0:
        q.put(merged)
    dist.destroy_process_group()


def test_sharding_two_ranks_gloo():
    import torch.multiprocessing as mp
    from linmt_b200 import shard
    c = synth.configs()["C1"]
    sents = c.sentences(23)
    parts = shard.partition(sents, 2, batch=4)
    assert sorted(parts[0] + parts[1]) == list(range(23))
    w = [sum(int(sents.steps[i]) + 1 for i in p) for p in parts]
    assert abs(w[0] - w[1]) <= 0.25 * max(w)
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + os.getpid() % 1000
    procs = [ctx.Process(target=_shard_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    merged = q.get(timeout=120)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert sorted(merged) == list(range(23))
    for i in range(23):
        assert merged[i] == (int(sents.ids[sents.off[i]:sents.off[i + 1]].sum()), int(sents.steps[i]))


def test_text_model_reader_and_cache(tmp_path):
    """Reference text model format -> blob through the library's reader, and the raw weight cache
    beside the text file: written on the first load, used while the text file is unchanged,
    ignored once it changes."""
    import os
    import time
    from linmt_b200 import modelfile
    d = synth.ModelDesc(2, 24, 37, 29, 1)
    blob = synth.make_blob(d, 9)
    path = str(tmp_path / "m.nmt")
    modelfile.write_model(path, d, blob)
    desc, got = modelfile.read_model(path, use_cache=False)
    assert (desc.L, desc.H, desc.V, desc.Vs, desc.feed_input) == (2, 24, 37, 29, 1)
    # the text carries 8 significant digits (src/deep_rnn.h:1991): values come back to fp32 rounding
    np.testing.assert_allclose(got, blob, rtol=2e-7, atol=0)
    assert not os.path.exists(path + ".linmtcache")
    _, first = modelfile.read_model(path, use_cache=True)
    assert os.path.exists(path + ".linmtcache")
    _, second = modelfile.read_model(path, use_cache=True)          # from the cache
    assert (first == got).all() and (second == got).all()
    # a changed text file (other weights, newer mtime) must not be served from the old cache
    blob2 = synth.make_blob(d, 10)
    modelfile.write_model(path, d, blob2)
    os.utime(path, (time.time() + 5, time.time() + 5))
    _, third = modelfile.read_model(path, use_cache=True)
    np.testing.assert_allclose(third, blob2, rtol=2e-7, atol=0)
    # the binary-body variant of the same file
    pathb = str(tmp_path / "mb.nmt")
    modelfile.write_model(pathb, d, blob, binary=True)
    _, gotb = modelfile.read_model(pathb, use_cache=False)
    assert (gotb == blob).all()
    with pytest.raises(RuntimeError):
        modelfile.read_model(str(tmp_path / "missing.nmt"))


def test_cpp_decoder_sentence_class_reports_init_errors(cpp_caller, tmp_path):
    """A C++ caller of DecoderSentence::Init / Process (src/decoder_sentence.h:40-41) compiles against
    include/linmt_decoder_sentence.hpp; a bad config is an error return with the reference's message, not
    an exit from inside the library."""
    import subprocess
    r = subprocess.run([cpp_caller, str(tmp_path / "none.config"), "in", "out"], capture_output=True, text=True)
    assert r.returncode == 2 and "does not exist" in r.stderr
    cfg = tmp_path / "a.config"
    cfg.write_text('param="--beam-size" value="4"\n')
    r = subprocess.run([cpp_caller, str(cfg), "in", "out"], capture_output=True, text=True)
    assert r.returncode == 2 and "--nmt-model" in r.stderr


def test_multi_device_job_order_and_errors(cuda_lib):
    """Handles on several devices: argument checks that need no GPU."""
    from linmt_b200 import _lib
    d = _lib.ModelDescC(1, 8, 20, 10, 1)
    o = _lib.OptionsC()
    cuda_lib.linmt_default_options(C.byref(o))
    blob = synth.make_blob(synth.ModelDesc(1, 8, 20, 10, 1), 0)
    arr = (C.c_void_p * 1)(blob.ctypes.data)
    h = C.c_void_p()
    devs = np.array([0, 1, 0], np.int32)
    rc = cuda_lib.linmt_create_from_weights_on(C.byref(d), arr, 1, blob.size, C.byref(o), devs.ctypes.data_as(C.c_void_p), 3, C.byref(h))
    assert rc == 1 and b"twice" in cuda_lib.linmt_last_error(None)
    assert cuda_lib.linmt_device_count(None) == 0


def test_bench_reference_arm_prints_the_contract_line():
    """`bench.py --impl reference` needs no GPU: it times the CPU restatement in the reference's loop shape and
    prints ONE JSON line with the same metric, unit and direction as the main arm, marked `impl: reference`, with
    a `cpu_baseline` that describes the run and an `e2e` that repeats the value with no copies."""
    import json
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    out = subprocess.run([sys.executable, os.path.join(root, "bench.py"), "--impl", "reference", "--workload", "C1",
                          "--steps", "1", "--warmup", "0"], capture_output=True, text=True, timeout=600, cwd=root)
    assert out.returncode == 0, out.stderr[-2000:]
    lines = [ln for ln in out.stdout.splitlines() if ln.strip()]
    assert len(lines) == 1, lines
    d = json.loads(lines[0])
    assert d["impl"] == "reference" and d["unit"] == "tokens/s" and d["higher_is_better"] is True
    assert d["metric"].startswith("decoded target tokens/sec") and d["value"] > 0 and d["gpu_launches"] == 0
    cb = d["cpu_baseline"]
    assert cb["kind"] in ("port", "reference") and cb["cores"] >= 1 and cb["sample"] and cb["value"] == d["value"]
    e = d["e2e"]
    assert e["value"] == d["value"] and e["unit"] == d["unit"] and e["h2d_bytes_per_step"] == 0 and e["d2h_bytes_per_step"] == 0
    assert d["config"]["workload"].startswith("C1")
