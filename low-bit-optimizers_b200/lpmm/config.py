"""Quantization configuration tree.

Mirrors the interface of the reference's ``lpmm/config.py`` -- ``get_config(None | path)``
returns a node tree read as ``cfg.QUANT.M.BITS``, ``cfg.QUANT.SQM.SCALE_TYPE.DEFAULT`` and so on
(defaults: config.py:7-79; YAML merge with ``BASE`` chaining: config.py:82-94) -- without
depending on yacs.  The node class supports what the optimizers and checkpoints need: attribute
and item access, ``clone``, ``defrost``/``freeze``, ``merge_from_file``, ``str`` and pickling.

Differences, on purpose: the reference prints the whole tree and writes ``./lpmm_config.txt`` on
every optimizer construction (config.py:190-196).  Here that happens only when the environment
variable ``LPMM_DUMP_CONFIG=1`` is set.  The argparse override block of the reference
(config.py:97-178) is research-script glue and is not provided.
"""
import copy
import os

import yaml

from .utils import get_rank


class ConfigNode(dict):
    """A dict whose keys read as attributes; nested dicts become nodes."""

    def __init__(self, init=None, new_allowed=False):
        super().__init__()
        object.__setattr__(self, "_frozen", False)
        object.__setattr__(self, "_new_allowed", new_allowed)
        for k, v in (init or {}).items():
            dict.__setitem__(self, k, ConfigNode(v, new_allowed) if isinstance(v, dict) and not isinstance(v, ConfigNode) else v)

    # attribute protocol ---------------------------------------------------------------------
    def __getattr__(self, name):
        try:
            return self[name]
        except KeyError:
            raise AttributeError(name) from None

    def __setattr__(self, name, value):
        if self._frozen:
            raise AttributeError(f"config is frozen; cannot set {name}")
        dict.__setitem__(self, name, ConfigNode(value, True) if isinstance(value, dict) and not isinstance(value, ConfigNode) else value)

    # copying / pickling ---------------------------------------------------------------------
    def clone(self):
        return copy.deepcopy(self)

    def __deepcopy__(self, memo):
        out = ConfigNode(new_allowed=self._new_allowed)
        for k, v in self.items():
            dict.__setitem__(out, k, copy.deepcopy(v, memo))
        object.__setattr__(out, "_frozen", self._frozen)
        return out

    def __reduce__(self):
        return (_rebuild_node, (dict(self), self._new_allowed, self._frozen))

    # freezing -------------------------------------------------------------------------------
    def _set_frozen(self, flag):
        object.__setattr__(self, "_frozen", flag)
        for v in self.values():
            if isinstance(v, ConfigNode):
                v._set_frozen(flag)

    def defrost(self):
        self._set_frozen(False)

    def freeze(self):
        self._set_frozen(True)

    def is_frozen(self):
        return self._frozen

    # merging --------------------------------------------------------------------------------
    def merge_from_dict(self, other):
        for k, v in other.items():
            if isinstance(v, dict) and isinstance(self.get(k), ConfigNode):
                self[k].merge_from_dict(v)
            elif isinstance(v, dict):
                dict.__setitem__(self, k, ConfigNode(v, True))
            else:
                dict.__setitem__(self, k, v)

    def merge_from_file(self, path):
        with open(path, "r") as fh:
            self.merge_from_dict(yaml.safe_load(fh) or {})

    # printing -------------------------------------------------------------------------------
    def __str__(self):
        lines = []
        for k in sorted(self):
            v = self[k]
            if isinstance(v, ConfigNode):
                lines.append(f"{k}:")
                lines.extend("  " + ln for ln in str(v).split("\n"))
            else:
                lines.append(f"{k}: {v}")
        return "\n".join(lines)

    def __repr__(self):
        return f"ConfigNode({dict.__repr__(self)})"


def _rebuild_node(items, new_allowed, frozen):
    node = ConfigNode(new_allowed=new_allowed)
    for k, v in items.items():
        dict.__setitem__(node, k, v)
    object.__setattr__(node, "_frozen", frozen)
    return node


def _moment(bits, scale, quant, signed, enable=True, group=128, rounding="real-nearest"):
    return {
        "ENABLE": enable, "THRESHOLD": 4096, "EXCLUDE_SUFFIX": [""], "EXCLUDE_REGEX": [""], "BITS": bits,
        "SCALE_TYPE": {"DEFAULT": scale, "DEFAULT_ONLY": True},
        "QUANT_TYPE": {"DEFAULT": quant, "DEFAULT_ONLY": True},
        "ROUND_TYPE": rounding, "GROUP_SIZE": group, "SIGNED": signed,
    }


def default_tree():
    """The in-code defaults used for ``qconfig=None`` (reference config.py:7-79): both moments
    4-bit, group-128 scales; first moment signed 'nonlinear', second moment unsigned 'power-1'."""
    return ConfigNode({
        "BASE": [""],
        "QUANT": {
            "INIT_STATES": ["param"],
            "P": _moment(8, "group", "linear", True, enable=False, group=64, rounding="sr"),
            "G": {"ENABLE": False, "THRESHOLD": 4096},
            "M": _moment(4, "group", "nonlinear", True),
            "SQM": _moment(4, "group", "power-1", False),
            "DEBUG": {"TRUNCATED_RATE_STAT_ITER": False, "ROW_ABSMAX_STAT_ITER": False, "ROW_ABSMAX_STAT_EPOCH": False},
        },
        "TRAIN": {},
        "OUTPUT": ".",
        "TAG": "",
        "LOCAL_RANK": 0,
    }, new_allowed=True)


def _merge_file(config, cfg_file):
    """Merge a YAML file, first merging every file named in its ``BASE`` list
    (paths relative to the file; reference config.py:82-94)."""
    with open(cfg_file, "r") as fh:
        loaded = yaml.safe_load(fh) or {}
    for base in loaded.get("BASE", [""]) or [""]:
        if base:
            _merge_file(config, os.path.join(os.path.dirname(cfg_file), base))
    config.defrost()
    config.merge_from_dict(loaded)
    config.freeze()


def get_config(args=None):
    """``None`` -> defaults; ``str`` -> defaults merged with that YAML file."""
    config = default_tree()
    if isinstance(args, str):
        _merge_file(config, args)
    elif isinstance(args, ConfigNode):
        config = args.clone()
    elif args is not None:
        raise TypeError("qconfig must be None, a path to a YAML file, or a ConfigNode "
                        "(argparse-namespace overrides of the reference are not provided)")
    config.freeze()
    if os.environ.get("LPMM_DUMP_CONFIG") == "1" and get_rank() == 0:
        print(config)
        with open(os.path.join(config.OUTPUT or ".", "lpmm_config.txt"), "w") as fout:
            fout.write(str(config))
    return config


CONFIG_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "configs")
