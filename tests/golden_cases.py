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
    "adamw_8bit": ("AdamW", dict(qconfig="default_8b.yml", **HYPER), [(72, 64), (4097,), (5000, 1)]),
    "adamw_5bit": ("AdamW", dict(qconfig="default_5b.yml", **HYPER), [(70, 61), (4100,)]),
    "adamw_m_group_512": ("AdamW", dict(qconfig="1st_moment_group_512.yml", **HYPER), [(72, 64), (4097,), (9000,)]),
    "adamw_m_group_4096": ("AdamW", dict(qconfig="1st_moment_group_4096.yml", **HYPER), [(70, 61), (10000,), (5000, 1)]),
    "sgd_8bit": ("SGD", dict(lr=1e-2, momentum=0.9, weight_decay=1e-4, qconfig="default_8b.yml"), [(72, 64), (4097,)]),
    "sgd_group_1024": ("SGD", dict(lr=1e-2, momentum=0.9, weight_decay=0.0, qconfig="1st_moment_group_1024.yml"),
                       [(5000,), (6, 700)]),
    "adamw_2nd_only_rank1": ("AdamW", dict(qconfig="2nd_moment_only_default.yml", **HYPER),
                             [(72, 64), (4097,), (100,), (2, 3, 32, 32)]),
    "adamw_2nd_only_group": ("AdamW", dict(qconfig="2nd_moment_only_group_128.yml", **HYPER), [(70, 61), (5000,)]),
    "adamw_override": ("AdamW", dict(qconfig="default.yml", **HYPER), [(72, 64), (3000,), (5000,), (50, 40)]),
}
# override_quantize_enable calls made before the first step: case -> [(parameter index, enable)]
OVERRIDES = {"adamw_override": [(0, False), (1, True), (3, True)]}
THRESHOLD = 4096

# Code width and first-moment group size of each case's configuration; names of its two maps in the
# qmaps fixture ('m' / 'v': the 4-bit maps; 'nonlinear_<b>' / 'power1_<b>': the wider ones).
def layout(name):
    cfg = CASES[name][1].get("qconfig")
    bits, m_gp = 4, 128
    if isinstance(cfg, str):
        if cfg.startswith("default_") and cfg.endswith("b.yml"):
            bits = int(cfg[len("default_"):-len("b.yml")])
        if cfg.startswith("1st_moment_group_"):
            m_gp = int(cfg[len("1st_moment_group_"):-len(".yml")])
    v_scale = "group" if cfg is None or cfg == "2nd_moment_only_group_128.yml" else "rank1"
    maps = ("m", "v") if bits == 4 else (f"nonlinear_{bits}", f"power1_{bits}")
    return dict(bits=bits, m_gp=m_gp, v_scale=v_scale, maps=maps)
