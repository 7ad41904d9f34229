"""CPU tests of the boundary: the shared library loads without a GPU, exports every symbol the
header declares, and the host-side mirror of the reference API behaves (no compute calls here)."""
import os
import re

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "fpq_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(fpq_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    from fpq_b200 import _cabi

    lib = _cabi.lib()
    names = declared_symbols()
    assert len(names) >= 13
    for n in names:
        assert hasattr(lib, n), f"{n} is declared in include/fpq_b200.h but not exported"
    assert sorted(_cabi.exported_symbols()) == names, "ctypes signatures and header are out of step"
    assert lib.fpq_version() >= 100
    assert isinstance(lib.fpq_last_error(), bytes)


def test_every_declaration_cites_the_reference():
    text = open(os.path.join(ROOT, "include", "fpq_b200.h")).read()
    for name in declared_symbols():
        if name in ("fpq_version", "fpq_last_error", "fpq_check_device", "fpq_cholesky_workspace_floats"):
            continue
        head = text[: text.index(f" {name}(")]
        comment = re.sub(r"[\s*]+", " ", head[head.rindex("/*"):])      # undo the comment's line breaks
        assert re.search(r"\.py:\d+", comment) or "no counterpart in the reference" in comment, name


def test_no_cpu_fallback():
    from fpq_b200 import ops

    with pytest.raises(RuntimeError, match="no CPU path"):
        ops.quantize(torch.zeros(4, 64), "mxfp4", 32)
    with pytest.raises(RuntimeError, match="no CPU path"):
        ops.rotate_hadamard(torch.zeros(4, 64), 32)


def test_product_never_imports_the_oracle():
    pkg = os.path.join(ROOT, "fp-quant_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h")):
                src = open(os.path.join(dirpath, f)).read()
                assert not re.search(r"^\s*(from|import)\s+oracle\b", src, flags=re.M), os.path.join(dirpath, f)


def test_config_validation_mirrors_reference_errors():
    from fpq_b200.fp_quant import FPQuantConfig, FPQuantDtype, validate_config

    validate_config(FPQuantConfig(forward_dtype=FPQuantDtype.MXFP4, forward_method="abs_max",
                                  backward_dtype=FPQuantDtype.BF16, hadamard_group_size=32))
    bad = [
        dict(forward_dtype=FPQuantDtype.NVFP4, forward_method="quest", backward_dtype=FPQuantDtype.BF16),
        dict(forward_dtype=FPQuantDtype.NVFP4, forward_method="abs_max", backward_dtype=FPQuantDtype.BF16,
             hadamard_group_size=8),
        dict(forward_dtype=FPQuantDtype.MXFP4, forward_method="abs_max", backward_dtype=FPQuantDtype.BF16,
             hadamard_group_size=16),
        dict(forward_dtype=FPQuantDtype.MXFP8, backward_dtype=FPQuantDtype.BF16),
        dict(forward_dtype=FPQuantDtype.NVFP4, forward_method="abs_max", backward_dtype=FPQuantDtype.MXFP4),
    ]
    for kw in bad:
        with pytest.raises(ValueError):
            validate_config(FPQuantConfig(**kw))


def test_rotation_classifier():
    from fpq_b200.fp_quant.module.linear import get_gsr_matrix, get_hadamard_matrix, get_identity_matrix
    from fpq_b200.rotation import classify_rotation

    cpu = torch.device("cpu")
    for g in (16, 32, 64, 128):
        assert classify_rotation(get_hadamard_matrix(g, torch.bfloat16, cpu)) == ("hadamard", g)
        assert classify_rotation(get_hadamard_matrix(g, torch.float32, cpu)) == ("hadamard", g)
        assert classify_rotation(get_identity_matrix(g, torch.bfloat16, cpu)) == ("identity", g)
        assert classify_rotation(get_gsr_matrix(g, torch.bfloat16, cpu)) == ("dense", g)


def test_replace_with_fp_quant_linear_on_meta():
    from torch import nn

    from fpq_b200.fp_quant import FPQuantConfig, FPQuantDtype, FPQuantLinear, replace_with_fp_quant_linear

    model = nn.Sequential()
    model.add_module("body", nn.Sequential(nn.Linear(64, 128, bias=False), nn.ReLU(), nn.Linear(128, 64)))
    model.add_module("lm_head", nn.Linear(64, 32))
    cfg = FPQuantConfig(forward_dtype=FPQuantDtype.NVFP4, forward_method="abs_max", backward_dtype=FPQuantDtype.BF16,
                        hadamard_group_size=16)
    model, replaced = replace_with_fp_quant_linear(model, cfg)
    assert replaced
    assert isinstance(model.body[0], FPQuantLinear) and isinstance(model.body[2], FPQuantLinear)
    assert isinstance(model.lm_head, nn.Linear) and not isinstance(model.lm_head, FPQuantLinear)
    assert model.body[0].qweight.shape == (128, 32) and model.body[0].scales.shape == (128, 4)
    assert model.body[0].qweight.device.type == "meta" and model.body[0].source_cls is nn.Linear
    assert set(model.body[2].state_dict()) >= {"weight", "dqweight", "bias", "qweight", "scales", "weight_global_scale",
                                               "act_global_scale", "forward_hadamard_matrix",
                                               "backward_hadamard_matrix"}


def test_padded_scale_shape():
    from fpq_b200 import ops

    assert ops.padded_scale_shape(1, 1) == (128, 4)
    assert ops.padded_scale_shape(128, 128) == (128, 128)
    assert ops.padded_scale_shape(130, 6) == (256, 8)
