"""Maps a golden case (reference-oracle vocabulary) to this build's mask/score vocabulary."""
from cases import make_doc_ids, slopes_for


def oracle_kwargs(c):
    kw = dict(sm_scale=c["sm_scale"])
    if c.get("docs"):
        kw.update(mask_kind="document", doc_ids=make_doc_ids(c))
    elif c.get("stride"):
        kw.update(mask_kind="s2", window=c["window"], stride=c["stride"])
    elif c.get("window") and c.get("causal"):
        kw.update(mask_kind="sliding_window_causal", window=c["window"])
    elif c.get("window"):
        kw.update(mask_kind="sliding_window", window=c["window"])
    elif c.get("causal"):
        kw.update(mask_kind="causal")
    if c.get("alibi"):
        kw.update(score_kind="alibi", alibi_slopes=slopes_for(c))
    if c.get("softcap"):
        kw.update(score_kind="softcap", cap=c["softcap"])
    return kw
