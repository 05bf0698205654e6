"""UNK post-processing (host string code, no GPU): the C++ implementation behind
python_unk_init / python_unk_do_job against the line-by-line restatement in oracle/unk_oracle.py
and against hand-worked answers."""
from __future__ import annotations

import random

import pytest

from oracle.unk_oracle import UnkOracle

DICT = {"haus": "house", "katze": "cat", "$number": "NUM", "gro@@": "big", "stadt": "city"}
STOP = {"der", "die", "das", ","}
ENDP = {".", "!", "?"}


@pytest.fixture(scope="module")
def unk(tmp_path_factory):
    from linmt_b200 import unk as unk_mod
    d = tmp_path_factory.mktemp("unk")
    (d / "dict.txt").write_text("".join(f"{k} ||| {v} ||| 1.0\n" for k, v in DICT.items()))
    (d / "stop.txt").write_text("".join(f"STOP\t{w}\n" for w in sorted(STOP)))
    (d / "punct.txt").write_text("".join(f"ENDPUNCT\t{w}\n" for w in sorted(ENDP)) + "OTHER\t;\n")
    cfg = d / "unk.config"
    cfg.write_text('# comment\nparam="--phrase-table" value="%s"\nparam="--stopword" value="%s"\n'
                   'param="--end-punct" value="%s"\n' % (d / "dict.txt", d / "stop.txt", d / "punct.txt"))
    p = unk_mod.PostProcessUnks()
    p.Init(str(cfg))
    unk_mod.unk_init(str(cfg))
    return p, unk_mod, UnkOracle(DICT, STOP, ENDP, emit_oov=True)


def line(words, align, scores, score="-1.5", unk_align=""):
    return f"{words} |||| {score} |||| {align} |||| {unk_align} |||| {scores}"


def test_hand_worked_cases(unk):
    p, mod, _ = unk
    # dictionary hit through the viterbi alignment
    assert mod.unk_do_job("das haus ist rot", line("the <UNK> is red", "0 1 2 3", "1/0/0/0 0/1/0/0 0/0/1/0 0/0/0/1")) == "the house is red"
    # out-of-vocabulary source word is copied in angle brackets
    assert mod.unk_do_job("das boot ist rot", line("the <UNK> is red", "0 1 2 3", "1/0/0/0 0/1/0/0 0/0/1/0 0/0/0/1")) == "the <boot> is red"
    # aligned to a stopword: the best-scored content word is used instead (position 1)
    assert mod.unk_do_job("der haus", line("<UNK> x", "0 1", "0.6/0.4 0/1")) == "house x"
    # generalization label filled from the source line's list, by alignment
    src = "er zahlt $number euro |||| {2 ||| 2 ||| 42 ||| $number ||| x}"
    assert mod.unk_do_job(src, line("he pays $number euros", "0 1 2 3", "1/0/0/0 0/1/0/0 0/0/1/0 0/0/0/1")) == "he pays 42 euros"
    # repeated words, repeated end punctuation
    assert mod.unk_do_job("a b c d e", line("x x y . . !", "0 1 2 3 4 4", "1/0/0/0/0 " * 6)) == "x y ."
    # fewer than five fields: nothing to work with -> first field is returned as is
    assert mod.unk_do_job("a b", "x y |||| -1.0") == "x y"
    assert mod.unk_do_job("a b", "x y") == ""
    assert mod.unk_do_job("", "x") == ""
    # sentence segmentation rule: source ends with "," -> a final "." becomes ","
    assert mod.unk_do_job("a ,", line("x .", "0 1", "1/0 0/1")) == "x ,"


def test_whole_line_keeps_fields(unk):
    p, _, ora = unk
    t = line("the <UNK>", "0 1", "1/0 0/1", score="-3.25", unk_align="1")
    got = p.Process("das haus", t)
    assert got == "the house |||| -3.25 |||| 0 1 |||| 1 |||| 1/0 0/1"
    assert got == ora.process("das haus", t)


def _random_case(rng):
    src_vocab = ["der", "die", "das", ",", "haus", "katze", "stadt", "boot", "gro@@", "$number", "$time", "$loc", "$NMT_a1",
                 "x", "y", ".", "$day", "$location"]
    tgt_vocab = ["<UNK>", "<UNK>", "the", "a", "x", "y", ".", "!", "$number", "$time", "$loc", "$day", "big", "cat", ","]
    ns, nt = rng.randint(1, 8), rng.randint(1, 10)
    src = [rng.choice(src_vocab) for _ in range(ns)]
    tgt = [rng.choice(tgt_vocab) for _ in range(nt)]
    align = [rng.randint(-1, ns) for _ in range(nt)]          # -1 and ns are out of range on purpose
    scores = []
    for _ in range(nt):
        n = ns if rng.random() < 0.9 else max(1, ns - 1)      # sometimes a malformed score list
        scores.append("/".join("%.3f" % rng.choice([0.0, 0.1, 0.25, 0.25, 0.5, rng.random()]) for _ in range(n)))
    gens = ""
    if rng.random() < 0.6:
        for pos, w in enumerate(src):
            if w in ("$number", "$time", "$loc", "$day", "$location") and rng.random() < 0.8:
                gens += "{%d ||| %d ||| G%d ||| %s ||| t}" % (pos, pos, pos, w)
            if w.startswith("$NMT_") and rng.random() < 0.8:
                gens += "{%d ||| %d ||| D%d ||| $dict ||| t}" % (pos, pos, pos)
    s = " ".join(src) + ((" |||| " + gens) if gens else "")
    t = line(" ".join(tgt), " ".join(map(str, align)), " ".join(scores))
    return s, t


def test_random_lines_match_restatement(unk):
    p, mod, ora = unk
    rng = random.Random(7)
    for _ in range(3000):
        s, t = _random_case(rng)
        want = ora.process(s, t)
        assert p.Process(s, t) == want, (s, t)
        assert mod.unk_do_job(s, t) == ora.do_job(s, t), (s, t)


def test_rm_oov_mode(tmp_path):
    from linmt_b200 import unk as unk_mod
    (tmp_path / "d").write_text("haus ||| house ||| 1\n")
    (tmp_path / "s").write_text("S\tder\n")
    (tmp_path / "e").write_text("ENDPUNCT\t.\n")
    cfg = tmp_path / "c"
    cfg.write_text('param="--phrase-table" value="%s"\nparam="--stopword" value="%s"\nparam="--end-punct" value="%s"\n'
                   'param="--rm-oov-mode" value="1"\n' % (tmp_path / "d", tmp_path / "s", tmp_path / "e"))
    p = unk_mod.PostProcessUnks()
    p.Init(str(cfg))
    assert p.Process("das boot", line("the <UNK>", "0 1", "1/0 0/1")).split(" |||| ")[0] == "the"
    with pytest.raises(RuntimeError):
        unk_mod.PostProcessUnks().Init(str(tmp_path / "missing.config"))
