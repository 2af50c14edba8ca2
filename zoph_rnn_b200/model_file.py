"""Writer for the reference's text weight file ("model.nn"), used to round-trip seeded models through
the reference's own format (layout: src/model.hpp:2015-2088; header: src/add_model_info.h:7-9; one matrix =
`rows` lines of `cols` numbers followed by a blank line, src/Eigen_Util.h:115-163)."""
import numpy as np

from .synth import tensor_spec


def default_vocab(cfg):
    """(source words, target words) with the reference's reserved entries: source id 0 is <UNK>
    (src/input_file_prep.h:328-341); target ids 0, 1, 2 are <START>, <EOF>, <UNK> (:346-348)."""
    src = ["<UNK>"] + [f"s{i}" for i in range(1, cfg["V_src"])] if not cfg["lm"] else []
    tgt = ["<START>", "<EOF>", "<UNK>"] + [f"t{i}" for i in range(3, cfg["V_tgt"])]
    return src, tgt[:cfg["V_tgt"]]


def write_model_nn(path, cfg, tensors, precision=9, src_words=None, tgt_words=None):
    """cfg: dict (synth.make_cfg); tensors: flat column-major float32 arrays in weight-file order.
    The header's attention flag is 0/1 (the reference has a single attention model)."""
    dsrc, dtgt = default_vocab(cfg)
    src_words = dsrc if src_words is None else src_words
    tgt_words = dtgt if tgt_words is None else tgt_words
    spec = tensor_spec(cfg)
    assert len(spec) == len(tensors)
    with open(path, "w") as f:
        hdr = [cfg["num_layers"], cfg["H"], cfg["V_tgt"], cfg["V_src"] if not cfg["lm"] else 0,
               1 if cfg["attention"] else 0, 1 if cfg["feed_input"] else 0, 0, 0, 0]
        f.write(" ".join(str(int(x)) for x in hdr) + "\n")
        f.write("=" * 44 + "\n")
        if not cfg["lm"]:
            for i in range(cfg["V_src"]):
                f.write(f"{i} {src_words[i]}\n")
            f.write("=" * 44 + "\n")
        for i in range(cfg["V_tgt"]):
            f.write(f"{i} {tgt_words[i]}\n")
        f.write("=" * 44 + "\n")
        fmt = "%." + str(precision) + "g"
        for (_, r, c), t in zip(spec, tensors):
            m = np.asarray(t, dtype=np.float32).reshape(c, r).T  # column-major -> (rows, cols)
            np.savetxt(f, m, fmt=fmt, delimiter=" ")
            f.write("\n")
