"""Pipeline layouts: which layers each (virtual) pipeline stage holds.

Two user-facing spellings, both from the reference:

* ``--pipeline-model-parallel-layout "Et*3|(tt|)*29,m|L"``: stages separated by ``|``; ``E`` embedding, ``t`` one
  transformer layer, ``m`` one multi-token-prediction layer, ``L`` the loss; ``x*n`` repeats a symbol and ``(...)*n`` a
  group; commas are cosmetic (docs/source/get_started/optimization_guide.md:156-169). Stages are listed for virtual
  stage 0 of every pipeline rank first, then virtual stage 1 of every rank, and so on.
* ``--custom-pipeline-layers 8,7,7,8`` (layers per pipeline rank) or ``--custom-virtual-pipeline-layers`` (layers per
  virtual stage, same order as above); the reference turns these into a layout string
  (loongforge/utils/utils.py:153-247, loongforge/train/validators.py:446-517).

The model builder only needs the number of transformer layers per virtual stage; this module produces that list and
checks what the rest of the framework assumes: embedding on the first stage, loss (and the MTP layers) on the last.
"""
from __future__ import annotations

import re
from typing import List, Optional, Sequence

_SYMBOLS = set("EtmL")


def expand_layout(layout: str) -> List[str]:
    """``"Et*3|(tt|)*2,m,L"`` -> ``["Ettt", "tt", "tt", "mL"]``."""
    s = layout.replace(" ", "")
    group = re.compile(r"\(([^()]*)\)\*(\d+)")
    while True:  # innermost groups first
        s2 = group.sub(lambda m: m.group(1) * int(m.group(2)), s)
        if s2 == s:
            break
        s = s2
    if "(" in s or ")" in s:
        raise ValueError(f"unbalanced or unrepeated parentheses in pipeline layout {layout!r}")
    s = re.sub(r"([EtmL])\*(\d+)", lambda m: m.group(1) * int(m.group(2)), s)
    s = s.replace(",", "")
    bad = set(s) - _SYMBOLS - {"|"}
    if bad:
        raise ValueError(f"unknown symbols {sorted(bad)} in pipeline layout {layout!r}")
    stages = s.split("|")
    if stages and stages[-1] == "" and s.endswith("|"):
        stages = stages[:-1]  # a trailing separator (e.g. from "(tt|)*n") closes the last stage, it does not open one
    return stages


def layers_per_virtual_stage(layout: str, pp: int, vpp: int = 1, *, num_layers: Optional[int] = None,
                             mtp_num_layers: int = 0) -> List[int]:
    """Transformer-layer count of virtual stage ``v * pp + pp_rank`` for every (v, pp_rank)."""
    stages = expand_layout(layout)
    n = pp * max(vpp, 1)
    if len(stages) != n:
        raise ValueError(f"pipeline layout has {len(stages)} stages; pp x virtual stages = {n}")
    if "E" not in stages[0] or any("E" in st for st in stages[1:]):
        raise ValueError("the embedding (E) belongs to the first stage, exactly once")
    if "L" not in stages[-1] or any("L" in st for st in stages[:-1]):
        raise ValueError("the loss (L) belongs to the last stage, exactly once")
    m_total = sum(st.count("m") for st in stages)
    if m_total != stages[-1].count("m"):
        raise NotImplementedError("multi-token-prediction layers (m) run on the stage that computes the loss; "
                                  "put them into the last stage of the layout")
    if m_total not in (0, mtp_num_layers):
        raise ValueError(f"layout lists {m_total} MTP layers, the model has {mtp_num_layers}")
    counts = [st.count("t") for st in stages]
    if num_layers is not None and sum(counts) != num_layers:
        raise ValueError(f"pipeline layout holds {sum(counts)} transformer layers, the model has {num_layers}")
    return counts


def split_rank_layers_over_virtual_stages(per_rank: Sequence[int], vpp: int) -> List[int]:
    """Layers per pipeline RANK -> layers per virtual stage: a rank's q*v + r layers go to its v chunks as r chunks of
    q + 1 (the later ones) and v - r chunks of q, like the reference's conversion."""
    pp, v = len(per_rank), max(vpp, 1)
    out = [0] * (pp * v)
    for r, nl in enumerate(per_rank):
        q, rem = divmod(nl, v)
        for c in range(v):
            out[c * pp + r] = q if c < v - rem else q + 1
    return out


def layout_from_counts(counts: Sequence[int], mtp_num_layers: int = 0) -> str:
    """Inverse of :func:`layers_per_virtual_stage` for plain layouts (what the reference logs and stores)."""
    stages = ["t" * c for c in counts]
    stages[0] = "E" + stages[0]
    stages[-1] = stages[-1] + "m" * mtp_num_layers + "L"
    return "|".join(stages)


def resolve_stage_layers(num_layers: int, pp: int, vpp: int = 1, *, layout: Optional[str] = None,
                         custom_pipeline_layers: Optional[Sequence[int]] = None,
                         custom_virtual_pipeline_layers: Optional[Sequence[int]] = None,
                         mtp_num_layers: int = 0) -> Optional[List[int]]:
    """The one entry point: per-virtual-stage layer counts from whichever spelling was given (None = even split)."""
    given = [x for x in (layout, custom_pipeline_layers, custom_virtual_pipeline_layers) if x]
    if len(given) > 1:
        raise ValueError("give only one of the pipeline layout, custom pipeline layers, custom virtual pipeline layers")
    v = max(vpp or 1, 1)
    if layout:
        return layers_per_virtual_stage(layout, pp, v, num_layers=num_layers, mtp_num_layers=mtp_num_layers)
    if custom_virtual_pipeline_layers:
        counts = list(custom_virtual_pipeline_layers)
        if len(counts) != pp * v:
            raise ValueError(f"{len(counts)} virtual-stage layer counts for pp x virtual stages = {pp * v}")
    elif custom_pipeline_layers:
        if len(custom_pipeline_layers) != pp:
            raise ValueError(f"{len(custom_pipeline_layers)} pipeline-stage layer counts for pp = {pp}")
        counts = split_rank_layers_over_virtual_stages(custom_pipeline_layers, v)
    else:
        return None
    if sum(counts) != num_layers:
        raise ValueError(f"custom pipeline layers sum to {sum(counts)}, the model has {num_layers}")
    return counts
