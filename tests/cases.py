"""The seeded cases the golden vectors were generated from (must mirror
tests/golden/make_golden.py)."""
from locks import synth

GQA_CASES = {
    "gqa_c0": dict(seed=1234, shape=synth.CONFIG0, seq_lens=[4097],
                   max_reqs=1, keep_blocks=48, combine="nrm", budget=None),
    "gqa_ragged": dict(
        seed=99,
        shape=synth.GqaShape(n_layers=2, n_kv=2, G=8, budget_pages=8,
                             sink_pages=1, window_pages=2, n_needles=2),
        seq_lens=[37, 530, 1203, 16 * 40], max_reqs=6, keep_blocks=20,
        combine="nrm", budget=None),
    "gqa_maxfrac": dict(
        seed=5,
        shape=synth.GqaShape(n_layers=1, n_kv=4, G=2, budget_pages=0,
                             sink_pages=2, window_pages=1, n_needles=2),
        seq_lens=[911, 64], max_reqs=2, keep_blocks=8, combine="max",
        budget=0.15),
}

MLA_CASES = {
    "mla_small": dict(seed=21,
                      shape=synth.MlaShape(n_layers=1, budget_pages=24,
                                           sink_pages=1, window_pages=4),
                      seq_lens=[777, 2048 + 5, 300], rank=8),
}


def make_gqa(name, device="cpu"):
    c = GQA_CASES[name]
    return synth.make_gqa_case(c["seed"], c["shape"], c["seq_lens"],
                               device=device), c


def make_mla(name, device="cpu"):
    c = MLA_CASES[name]
    return synth.make_mla_case(c["seed"], c["shape"], c["seq_lens"],
                               device=device, n_layers=1), c
