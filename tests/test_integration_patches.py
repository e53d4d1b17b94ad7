"""The Megatron-LM and fairseq patches are real ``git apply``-able diffs.  Their targets are not on this machine,
so each patch is applied to a stand-in tree rebuilt from its own pre-image (the context and removed lines of every
hunk, at the line numbers the hunk headers name): that checks the diff syntax, the hunk arithmetic and that the
added code calls functions the helper modules really export."""

import os
import re
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PATCHES = [
    ('planmoe_b200/examples/megatron/planmoe_megatron.diff', 'planmoe_b200.examples.megatron.planmoe_megatron'),
    ('planmoe_b200/examples/fairseq_moe/planmoe_fairseq.diff', 'planmoe_b200.examples.fairseq_moe.planmoe_fairseq'),
]


def _preimage(patch_text):
    """{path: text} with each hunk's pre-image placed at its stated start line (blank filler in between)."""
    files, cur, lines = {}, None, None
    for ln in patch_text.splitlines():
        if ln.startswith('--- a/'):
            cur = ln[6:]
            lines = files.setdefault(cur, [])
        elif ln.startswith('@@'):
            start = int(re.match(r'@@ -(\d+)', ln).group(1))
            while len(lines) < start - 1:
                lines.append('# filler')
        elif cur is not None and (ln.startswith(' ') or ln.startswith('-')) and not ln.startswith('---'):
            lines.append(ln[1:])
    return {k: '\n'.join(v) + '\n' for k, v in files.items()}


@pytest.mark.parametrize("patch,module", PATCHES)
def test_patch_applies_and_calls_existing_helpers(tmp_path, patch, module):
    text = open(os.path.join(ROOT, patch)).read()
    for path, body in _preimage(text).items():
        full = tmp_path / path
        full.parent.mkdir(parents=True, exist_ok=True)
        full.write_text(body)
    subprocess.run(['git', 'init', '-q'], cwd=tmp_path, check=True)
    res = subprocess.run(['git', 'apply', '--verbose', os.path.join(ROOT, patch)], cwd=tmp_path,
                         stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    assert res.returncode == 0, res.stdout
    import importlib
    helper = importlib.import_module(module)
    added = [ln[1:] for ln in text.splitlines() if ln.startswith('+') and not ln.startswith('+++')]
    short = module.rsplit('.', 1)[1]
    called = set(re.findall(short + r'\.(\w+)\(', '\n'.join(added)))
    called |= set(re.findall(r'import (\w+)$', '\n'.join(l for l in added if module in l), flags=re.M)) - {short}
    assert called, "the patch calls nothing"
    for name in called:
        assert hasattr(helper, name), name


def test_fairseq_helper_builds_the_layer_the_patch_describes(monkeypatch):
    """MOE=2: layer index 1 becomes a top-2, dynamic-capacity layer with one expert per rank; index 0 stays dense."""
    import types
    import torch
    from planmoe_b200.examples.fairseq_moe import planmoe_fairseq as pf
    monkeypatch.setenv('MOE', '2')
    monkeypatch.setenv('L_AUX_WT', '0.01')
    cfg = types.SimpleNamespace(decoder=types.SimpleNamespace(ffn_embed_dim=64))
    layer = types.SimpleNamespace(embed_dim=32, quant_noise=0, activation_fn=torch.nn.functional.gelu,
                                  activation_dropout_module=torch.nn.Identity(), ffn_layernorm=None)
    assert pf.build_ffn_for_layer(layer, pf.tag_layer_index(cfg, 0)) is None
    moe = pf.build_ffn_for_layer(layer, pf.tag_layer_index(cfg, 1))
    assert moe is not None and moe.gates[0].top_k == 1 or moe.gates[0].top_k == 2
    x = torch.randn(4, 6, 32, requires_grad=True)
    moe.train()
    y = pf.ffn_forward(moe, x)
    loss = pf.add_aux_loss(y.sum())
    loss.backward()
    assert x.grad is not None and torch.isfinite(loss)
