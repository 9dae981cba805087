"""The cases of tests/golden/make_python_golden.py, restated for the tests that replay them."""
HYPER = dict(lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.01)

CASES = {
    "adamw_rank1": ("AdamW", dict(qconfig="default.yml", **HYPER), [(64, 96), (96,)]),
    "adamw_group": ("AdamW", dict(qconfig=None, **HYPER), [(72, 64), (4097,), (127,)]),
    "adamw_rank1_ragged": ("AdamW", dict(qconfig="default.yml", **HYPER),
                           [(3, 3, 24, 24), (70, 61), (4097,), (127,), (4096,), (5000, 1)]),
    "adamw_factored": ("AdamW", dict(qconfig=None, factor_second_moment=True, **HYPER),
                       [(80, 64), (2, 3, 32, 32), (40, 8), (5000,)]),
    "sgd_momentum": ("SGD", dict(lr=1e-2, momentum=0.9, weight_decay=1e-4, qconfig=None), [(72, 64), (4097,), (100,)]),
    "sgd_nesterov": ("SGD", dict(lr=1e-2, momentum=0.8, dampening=0.0, nesterov=True, weight_decay=0.0, qconfig=None),
                     [(5000,), (6, 700)]),
}
THRESHOLD = 4096
