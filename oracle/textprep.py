"""TEST INFRASTRUCTURE ONLY: a plain-Python restatement of the reference's data preparation either side of the
forward path, used by tests/ to check the front end's integer files and output formatting.  Nothing in the product
imports this file.  Parity unpinned: the reference ships no fixtures for these routines and cannot be built here;
every function cites the reference lines it follows.
"""

MINIBATCH_MULT = 10  # src/input_file_prep.h:105


def read_vocab(model_path):
    """Header ints and the word -> id maps of a model.nn (src/input_file_prep.h:1981-2025; sequence models have the
    target section only, :2776-2790)."""
    with open(model_path) as f:
        header = [int(x) for x in f.readline().split()]
        f.readline()
        lm = header[3] <= 0
        maps = []
        for _ in range(1 if lm else 2):
            m = {}
            for line in f:
                if line.startswith("==="):
                    break
                parts = line.split()
                m[parts[1]] = int(parts[0])
            maps.append(m)
    src, tgt = ({}, maps[0]) if lm else (maps[0], maps[1])
    return header, src, tgt


def _lines(path):
    with open(path) as f:
        return [l.rstrip("\n") for l in f]


def _src_id(src, w):
    return src[w] if w in src else src.get("<UNK>", 0)  # src/input_file_prep.h:2238-2244


def _tgt_id(tgt, w):
    if w in tgt:
        return tgt[w]
    return tgt["<UNK>"] if "<UNK>" in tgt else tgt.get("<UNK>NULL", 0)  # :2315-2325


def _window_sort(data, minibatch):
    """Sort by total length inside windows of minibatch * 10 sentences (src/input_file_prep.h:2191-2204); ties keep
    file order (the reference's std::sort leaves them unspecified)."""
    win = minibatch * MINIBATCH_MULT
    cur = 0
    while cur < len(data):
        if cur + win <= len(data):
            data[cur:cur + win] = sorted(data[cur:cur + win], key=lambda d: len(d[0]) + len(d[1]))
            cur += win
        else:
            data[cur:] = sorted(data[cur:], key=lambda d: len(d[0]) + len(d[1]))
            break


def _fmt(ids):
    return "".join(f"{i} " for i in ids) + "\n"  # every id is followed by a blank (:2435-2441)


def integerize_nonlm(model_path, src_path, tgt_path, longest_sent, minibatch):
    """integerize_file_nonLM (src/input_file_prep.h:1958-2547).  Returns the text of the integer file."""
    _, src, tgt = read_vocab(model_path)
    sl, tl = _lines(src_path), _lines(tgt_path)
    assert len(sl) == len(tl)
    data = []
    for s, t in zip(sl, tl):
        s, t = s.split(), t.split()
        if not (len(s) + 1 >= longest_sent - 2 or len(t) + 1 >= longest_sent - 2):  # :2147
            data.append((s, t))
    if minibatch != 1:
        _window_sort(data, minibatch)
    if len(data) % minibatch:
        data = data[:len(data) - len(data) % minibatch]  # :2207-2213
    recs = []
    for s, t in data:
        si = [_src_id(src, w) for w in s][::-1]  # :2259
        ti = [_tgt_id(tgt, w) for w in t]
        recs.append([si, [-2] * len(si), [0] + ti, ti + [1]])  # :2276-2278, :2346-2347
    for cur in range(0, len(recs), minibatch):
        grp = recs[cur:cur + minibatch]
        ms = max(len(r[0]) for r in grp)
        mt = max(len(r[2]) for r in grp)
        for r in grp:  # :2374-2385
            pad = ms - len(r[0])
            r[0] = [-1] * pad + r[0]
            r[1] = [-1] * pad + r[1]
            r[2] = r[2] + [-1] * (mt - len(r[2]))
            r[3] = r[3] + [-1] * (mt - len(r[3]))
    return "".join(_fmt(r[0]) + _fmt(r[1]) + _fmt(r[2]) + _fmt(r[3]) for r in recs)


def integerize_lm(model_path, tgt_path, longest_sent, minibatch):
    """integerize_file_LM (src/input_file_prep.h:2743-2968)."""
    _, _, tgt = read_vocab(model_path)
    data = []
    for t in _lines(tgt_path):
        t = t.split()
        if not (len(t) + 1 >= longest_sent - 2):  # :2824
            data.append(([], t))
    if minibatch != 1:
        _window_sort(data, minibatch)
    recs = []
    for _, t in data:
        ti = [_tgt_id(tgt, w) for w in t]
        recs.append([[0] + ti, ti + [1]])
    for cur in range(0, len(recs), minibatch):
        grp = recs[cur:cur + minibatch]
        mt = max(len(r[0]) for r in grp)
        for r in grp:  # one -1 column more than the longest row (:2902)
            r[0] = r[0] + [-1] * (mt + 1 - len(r[0]))
            r[1] = r[1] + [-1] * (mt + 1 - len(r[1]))
    extra = minibatch - len(recs) % minibatch
    if extra != minibatch:  # complete the last minibatch with -1 rows (:2913-2930)
        width = len(recs[-1][0])
        recs += [[[-1] * width, [-1] * width] for _ in range(extra)]
    return "".join("\n\n" + _fmt(r[0]) + _fmt(r[1]) for r in recs)


def integerize_kbest(model_path, src_path, longest_sent, legacy=False):
    """integerize_file_kbest (src/input_file_prep.h:2970-3134)."""
    _, src, _ = read_vocab(model_path)
    out = []
    for s in _lines(src_path):
        s = s.split()[::-1]  # :3081
        if len(s) + 1 >= longest_sent - 2:
            continue
        ids = [_src_id(src, w) for w in s]
        if legacy:
            ids = [0] + ids
        out.append(ids)
    return "".join(_fmt(i) for i in out), out


def format_kbest_ints(hyps, print_score):
    """decoder::output_k_best_hypotheses (src/decoder.h:1413-1457): hyps = per sentence a list of (ids, score),
    best first.  Scores are printed with the stream's default 6 significant digits."""
    out = []
    for sent in hyps:
        out.append("------------------------------------------------\n")
        for ids, score in sent:
            if print_score:
                out.append("-Score: %s\n" % cxx_stream_float(score))
            out.append("".join(f"{i} " for i in ids) + "\n")
        out.append("\n")
    return "".join(out)


def format_unk_file(hyps):
    """The --UNK-decode file (src/decoder.h:1452-1459): one line per printed hypothesis; for every position j that
    holds <UNK> (id 2) the alignment stored at j + 1.  hyps = per sentence a list of (ids, alignments)."""
    out = []
    for sent in hyps:
        for ids, align in sent:
            out.append("".join(f"{align[j + 1]} " for j in range(len(ids)) if ids[j] == 2) + "\n")
    return "".join(out)


def unint(model_path, text, decoder=True):
    """unint_file (src/input_file_prep.h:3137-3205)."""
    _, _, tgt = read_vocab(model_path)
    rev = {v: k for k, v in tgt.items()}
    out = []
    for line in text.split("\n")[:-1] if text.endswith("\n") else text.split("\n"):
        if decoder and (line == "" or line[0] in "- "):
            out.append(line + "\n")
            continue
        out.append(" ".join(rev.get(int(x), "") for x in line.split()) + "\n")
    return "".join(out)


def cxx_stream_float(x):
    """What `std::ostream << x` prints with default flags: %g with 6 significant digits."""
    return "%g" % x
