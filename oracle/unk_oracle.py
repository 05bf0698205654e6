"""TEST INFRASTRUCTURE ONLY -- CPU restatement of the reference's UNK post-processing
(src/postprocess_unks.cc), the step its Python wrapper runs right after `python_decoder_do_job`.

PARITY UNPINNED: the reference ships no tests, fixtures or golden vectors for this code and cannot
be built here; this file follows the source line by line (citations below) and the product's C++
implementation (linmt_b200/csrc/unk_post.cpp) is compared with it on crafted and random cases.

Only tests/ may import this module.
"""
from __future__ import annotations

# labels whose target-side occurrence is filled from the generalization list of the source line
# (Processing, postprocess_unks.cc:458-516): target word -> (slot, label printed when nothing is found)
TARGET_LABELS = {
    "$number": "number", "$time": "time", "$date": "date", "$day": "day", "$psn": "person", "$loc": "location",
    "$location": "location", "$org": "organization", "$literal": "literal",
    **{f"$userdict{i}": f"userdict{i}" for i in range(1, 11)},
}
# field 3 of a generalization entry -> slot (postprocess_unks.cc:262-305)
ENTRY_SLOTS = dict(TARGET_LABELS, **{"$dict": "dict"})
# source words that the dictionary branch treats as labels (postprocess_unks.cc:389-407)
DICT_BRANCH_LABELS = set(TARGET_LABELS)
# source words FindUnStopword skips (postprocess_unks.cc:661-678): no $day, no $location
UNSTOP_SKIP = {"$number", "$time", "$date", "$psn", "$loc", "$org", "$literal", *[f"$userdict{i}" for i in range(1, 11)]}


def split_char(s: str, c: str):
    """BasicMethod::Split (utility_cc.cc:132-153): empty pieces dropped."""
    return [p for p in s.split(c) if p != ""]


def split_str(s: str, sep: str):
    """BasicMethod::SplitWithString (utility_cc.cc:157-176): a separator at position 0 is skipped,
    empty pieces in the middle are kept, nothing is added after a trailing separator."""
    out = []
    start = 0
    while start < len(s):
        idx = s.find(sep, start)
        if idx == 0:
            start += len(sep)
            continue
        if idx < 0:
            out.append(s[start:])
            break
        out.append(s[start:idx])
        start = idx + len(sep)
    return out


def clear_illegal(s: str) -> str:
    return s.replace("\r", "").replace("\n", "")


def c_atoi(s: str) -> int:
    """atoi: optional spaces, sign, digits; 0 if none."""
    s = s.lstrip(" \t")
    i, sign = 0, 1
    if i < len(s) and s[i] in "+-":
        sign = -1 if s[i] == "-" else 1
        i += 1
    j = i
    while j < len(s) and s[j].isdigit():
        j += 1
    return sign * int(s[i:j]) if j > i else 0


def c_atof(s: str) -> float:
    """atof rounded to float as the multimap<float,int> key does; longest numeric prefix."""
    import re
    import struct
    m = re.match(r"\s*[+-]?(\d+\.?\d*([eE][+-]?\d+)?|\.\d+([eE][+-]?\d+)?)", s)
    v = float(m.group(0)) if m else 0.0
    return struct.unpack("f", struct.pack("f", v))[0]


def ranked_positions(align_scores: str, n_src: int):
    """Positions by descending score; among equal scores the later position first (reverse
    iteration over a multimap filled in position order).  None on a length mismatch
    (postprocess_unks.cc:619-634, 644-659)."""
    scores = split_char(align_scores, "/")
    if len(scores) != n_src:
        return None
    keyed = [(c_atof(x), i) for i, x in enumerate(scores)]
    return [i for _, i in sorted(keyed, key=lambda t: (t[0], t[1]), reverse=True)]


def is_nmt_label(w: str) -> bool:
    return len(w) > 5 and w.startswith("$NMT_")


class UnkOracle:
    def __init__(self, dictionary, stopwords, end_puncts, emit_oov=True):
        self.dict = dict(dictionary)
        self.stop = set(stopwords)
        self.endp = set(end_puncts)
        self.emit_oov = emit_oov   # remove_oov_mode_ after the inversion of GeneralSettings (:104-108)

    # FindUnStopword, postprocess_unks.cc:644-690
    def find_unstopword(self, scores, src):
        order = ranked_positions(scores, len(src))
        if order is None:
            return -1
        for p in order:
            if src[p] not in self.stop and src[p] not in UNSTOP_SKIP:
                return p
        return -1

    # Processing, postprocess_unks.cc:220-613
    def process(self, line_source: str, line_translation: str) -> str:
        line_translation = clear_illegal(line_translation)
        line_source = clear_illegal(line_source)
        parts = split_str(line_source, " |||| ")
        line_source = parts[0]
        slots = {}
        if len(parts) == 2:
            g = parts[1]
            if len(g) >= 3 and g[0] == "{" and g[-1] == "}":
                for entry in split_str(g[1:-1], "}{"):
                    f = split_str(entry, " ||| ")
                    if len(f) == 5 and f[3] in ENTRY_SLOTS:
                        slots.setdefault(ENTRY_SLOTS[f[3]], {})[c_atoi(f[0])] = f[2]
        fields = split_str(line_translation, " |||| ")
        if len(fields) < 5:
            return line_translation
        src = split_char(line_source, " ")
        tgt = split_char(fields[0], " ")
        if tgt and tgt[-1] == "." and src and src[-1] == ",":
            tgt[-1] = ","
        score_fields = split_char(fields[4], " ")
        align = []
        import re
        for tok in fields[2].split():   # istream >> int: stops at the first token that is not an integer
            m = re.match(r"[+-]?\d+", tok)
            if not m:
                break
            align.append(int(m.group(0)))
            if m.end() != len(tok):
                break
        if len(tgt) != len(align):
            return line_translation
        out = ""
        gdict = slots.setdefault("dict", {})

        def scores_of(i):
            return score_fields[i] if i < len(score_fields) else ""

        def from_position(pos, unk_form):
            nonlocal out
            if pos == -1:
                out += " ."
            elif 0 <= pos < len(src):
                w = src[pos]
                if is_nmt_label(w):
                    if pos in gdict:
                        out += " " + gdict[pos]
                elif w in self.dict:
                    out += (" <UNK-" + self.dict[w] + ">") if unk_form else (" " + self.dict[w])
                elif self.emit_oov:
                    out += " <" + w + ">"

        for i, w in enumerate(tgt):
            a = align[i]
            if w == "<UNK>":
                if 0 <= a < len(src):
                    sw = src[a]
                    if is_nmt_label(sw):
                        if a in gdict:
                            out += " " + gdict[a]
                    elif sw in self.stop:
                        from_position(self.find_unstopword(scores_of(i), src), True)
                    elif sw in self.dict:
                        if sw not in DICT_BRANCH_LABELS:
                            out += " <UNK-" + self.dict[sw] + ">"
                        else:
                            from_position(self.find_unstopword(scores_of(i), src), False)
                    elif self.emit_oov:
                        out += " <" + sw + ">"
            elif w in TARGET_LABELS:
                # TargetIsGeneralization, postprocess_unks.cc:595-613
                slot = slots.setdefault(TARGET_LABELS[w], {})
                if a in slot:
                    out += " " + slot.pop(a)
                else:
                    order = ranked_positions(scores_of(i), len(src))
                    pos = -1
                    if order is not None:
                        for p in order:
                            if p in slot:
                                pos = p
                                break
                    if pos != -1:
                        out += " " + slot.pop(pos)
                    elif self.emit_oov:
                        out += " <" + w + ">"
            else:
                out += " " + w
        out = out.lstrip(" ")
        # consecutive identical words (:524-539)
        words = split_char(out, " ")
        kept, last = [], ""
        for x in words:
            if x == last:
                continue
            kept.append(x)
            last = x
        out = " ".join(kept)
        # consecutive identical bigrams (:541-562)
        w = split_char(out, " ")
        n = len(w)
        if n >= 4:
            out = w[0] + " " + w[1]
            last_bigram = out
            i = 3
            while i < n:
                cur = w[i - 1] + " " + w[i]
                if cur != last_bigram:
                    out += " " + w[i - 1]
                    last_bigram = w[i - 2] + " " + w[i - 1]
                else:
                    i += 1
                i += 1
            if n + 1 != i:
                out += " " + w[n - 1]
        # consecutive end punctuations (:565-588)
        w = split_char(out, " ")
        out = ""
        last_end = False
        for i, x in enumerate(w):
            if x in self.endp:
                if last_end:
                    continue
                last_end = True
            else:
                last_end = False
            if i != 0:
                out += " "
            out += x
        # "<UNK-...>" markers of the dictionary branch (:591-611)
        if "<UNK-" in out:
            out = out.replace("@@ ", "")
            w = split_char(out, " ")
            out = ""
            i = 0
            while i < len(w):
                x = w[i]
                if len(x) >= 6 and x.startswith("<UNK-") and x.endswith(">"):
                    sub = x[5:-1]
                    out += " " + sub
                    if i < len(w) - 1 and w[i + 1] in sub:
                        i += 1
                else:
                    out += " " + x
                i += 1
        out = out.lstrip(" ")
        for f in fields[1:]:
            out += " |||| " + f
        return out

    # python_unk_do_job, postprocess_unks.cc:724-752
    def do_job(self, src_sentence: str, translation: str) -> str:
        if src_sentence == "" or translation == "":
            return ""
        f = split_str(self.process(src_sentence, translation), " |||| ")
        return f[0] if len(f) > 1 else ""
