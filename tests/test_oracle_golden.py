"""The CPU oracle against fixtures produced by the reference's own code (tests/golden/make_golden.py)."""
import glob
import json
import os

import numpy as np
import pytest
import torch

from oracle import attention as oa
from oracle import bookkeeping as ob


@pytest.fixture(scope="module")
def book(golden_dir):
    with open(os.path.join(golden_dir, "bookkeeping.json")) as f:
        return json.load(f)


def test_patches_metadata(book):
    assert len(book["patches_metadata"]) > 50
    for c in book["patches_metadata"]:
        fn = ob.calc_patches_metadata if c["variant"] == "image" else ob.calc_cogvideox_patches_metadata
        args = (c["height"], c["width"], c["vae"], c["patch"], c["num_pipeline_patch"], c["sp_world"], c["sp_rank"])
        if "error" in c:
            with pytest.raises(ValueError):
                fn(*args)
        else:
            assert fn(*args) == c["result"], c


def test_rank_generator(book):
    for c in book["rank_generator"]:
        for tok, groups in c["groups"].items():
            got = ob.rank_generator_groups(c["tp"], c["sp"], c["pp"], c["cfg"], c["dp"], tok,
                                           rank_offset=c["rank_offset"])
            assert got == groups, (c, tok)
    for c in book["masked_orthogonal"]:
        assert ob.orthogonal_rank_groups(c["world"], c["sizes"], c["mask"]) == c["groups"]


def test_seq_parallel_groups(book):
    for c in book["seq_parallel_groups"]:
        ug, rg = ob.seq_parallel_rank_groups(c["ulysses"], c["ring"], len(c["ranks"]), c["ranks"],
                                             c["use_ulysses_low"])
        for rank, groups in c["per_rank"].items():
            mine_u = [g for g in ug if int(rank) in g]
            mine_r = [g for g in rg if int(rank) in g]
            assert mine_u == [groups["ulysses"]] and mine_r == [groups["ring"]], c


def test_comm_pool_enumeration(book):
    for c in book["rank_combinations"]:
        assert ob.rank_combinations(c["world"], base_num=c["base"]) == c["result"]
    for c in book["group_partitions"]:
        assert ob.group_partitions(c["ranks"]) == c["result"]


def test_slice_ranges(book):
    for c in book["range_to_indices"]:
        assert list(ob.range_to_indices_round(c["range"], c["total"])) == c["round"], c
        assert list(ob.range_to_indices_trunc(c["range"], c["total"])) == c["trunc"], c
    for c in book["gpu_metadata"]:
        got = ob.gpu_metadata(c["pp_rank"], c["pp_world"], c["tp_rank"], c["tp_world"])
        assert {k: list(v) for k, v in got.items()} == c["result"]


def test_tp_split_table(book):
    for c in book["tp_split_type"]:
        assert ob.tp_split_type(c["name"]) == c["result"], c


def test_migration_plans(book):
    for c in book["migration_plans"]:
        n = c["num_blocks"]
        s, e = ob.range_to_indices_trunc(c["new_pp"], n)
        linears = {i: [tuple(l) for l in c["linears"]] for i in range(n)}
        cached = {int(k): tuple(v) for k, v in c["cached"].items()}
        got = ob.needed_pieces(list(range(s, e)), linears, cached, tuple(c["target_tp"]), c["slice_bias"])
        assert got == c["pieces"], c["kind"]


def test_rope(golden_dir):
    with np.load(os.path.join(golden_dir, "rope.npz")) as f:
        for i in range(2):
            x, cos, sin = (torch.from_numpy(f[f"{n}{i}"]) for n in ("x", "cos", "sin"))
            assert torch.equal(oa.apply_rotary_emb(x, cos, sin), torch.from_numpy(f[f"y{i}"]))
            yb = oa.apply_rotary_emb(x.to(torch.bfloat16), cos, sin).float()
            assert torch.equal(yb, torch.from_numpy(f[f"yb{i}"]))


def _load_usp(path):
    with np.load(path) as f:
        d = {k: f[k] for k in f.files}
    spec = json.loads(str(d.pop("spec")))
    return spec, {k: torch.from_numpy(v) for k, v in d.items()}


@pytest.mark.parametrize("path", sorted(glob.glob(os.path.join(os.path.dirname(__file__), "golden", "usp_*.npz"))),
                         ids=lambda p: os.path.basename(p)[4:-4])
def test_usp_attention(path):
    spec, d = _load_usp(path)
    P, S = spec["world"], spec["s_loc"]
    strategy = spec["joint_strategy"]

    def shard(t, n):
        return [t[:, r * n:(r + 1) * n].contiguous() for r in range(P)]

    joint = dict(joint_qs=[d["jq"]] * P, joint_ks=[d["jk"]] * P, joint_vs=[d["jv"]] * P) if strategy != "none" else {}
    if not spec["kv_cache"]:
        outs = oa.usp_attention(shard(d["q"], S), shard(d["k"], S), shard(d["v"], S), spec["ulysses"], spec["ring"],
                                joint_strategy=strategy, **joint)
        for r in range(P):
            torch.testing.assert_close(outs[r], d[f"out_rank{r}"], rtol=1e-5, atol=1e-5)
        # and, by construction, USP equals plain attention over the un-sharded sequence
        if strategy == "none":
            full = oa.sdpa(d["q"], d["k"], d["v"])
        elif strategy == "rear":
            full = oa.sdpa(d["q"], torch.cat([d["k"], d["jk"]], 1), torch.cat([d["v"], d["jv"]], 1))
        else:
            full = oa.sdpa(d["q"], torch.cat([d["jk"], d["k"]], 1), torch.cat([d["jv"], d["v"]], 1))
        for r in range(P):
            local = outs[r][:, :S] if strategy != "front" else outs[r][:, spec["s_txt"]:]
            torch.testing.assert_close(local, full[:, r * S:(r + 1) * S], rtol=2e-5, atol=2e-5)
    else:
        # warm-up call == plain USP; the patch call attends to the stale buffer with patch 1's range replaced
        U = spec["ulysses"]
        outs = oa.usp_attention(shard(d["q"], S), shard(d["k"], S), shard(d["v"], S), U, spec["ring"],
                                joint_strategy=strategy, **joint)
        for r in range(P):
            torch.testing.assert_close(outs[r], d[f"out_warmup_rank{r}"], rtol=1e-5, atol=1e-5)
        n_patch, tok = 2, S // 2
        tok_start = [0, tok, 2 * tok]
        fq, fk, fv = (d[f"fresh_{n}"] for n in ("q", "k", "v"))
        H = spec["heads"]
        hpr = H // U
        for r in range(P):
            hs = slice(r * hpr, (r + 1) * hpr)
            # gathered K‖V of the warm-up step for this rank's heads (rank-major order, unchanged)
            cache = torch.cat([d["k"][:, :, hs], d["v"][:, :, hs]], dim=-1).clone()
            new_kv = torch.cat([fk[:, :, hs], fv[:, :, hs]], dim=-1)
            kv = oa.kv_cache_update(cache, new_kv, True, n_patch, 1, tok_start, slice_dim=1, ulysses_world=U,
                                    sequence_parallel=True)
            k_all, v_all = torch.chunk(kv, 2, dim=-1)
            def join(x, j):                      # text rows behind ("rear") or in front of the image rows
                return torch.cat([x, j] if strategy == "rear" else [j, x], dim=1)

            q_loc = join(fq[:, r * tok:(r + 1) * tok], d["jq"])
            q_g = torch.cat([join(fq[:, s * tok:(s + 1) * tok], d["jq"]) for s in range(P)], dim=1)[:, :, hs]
            k_g = join(k_all, d["jk"][:, :, hs])
            v_g = join(v_all, d["jv"][:, :, hs])
            ctx = oa.sdpa(q_g, k_g, v_g)  # (B, P*(tok+S_t), hpr, D): this rank's head slice, all ranks' rows
            rows = tok + spec["s_txt"]
            for dst in range(P):
                torch.testing.assert_close(ctx[:, dst * rows:(dst + 1) * rows], d[f"out_patch1_rank{dst}"][:, :, hs],
                                           rtol=2e-5, atol=2e-5)
            assert q_loc.shape[1] == rows


def test_pipefusion_oracle_stale_kv_order_matches_the_reference_run():
    """oracle/pipefusion.py models the stale K/V of a plan with Ulysses by a row order (warmup_cache_order) and
    patch writes at image-order positions. The kv-cache fixture was recorded from the reference's own
    CacheManager and operator on two ranks: the model must reproduce its patch-step outputs."""
    from oracle import pipefusion as opf
    path = os.path.join(os.path.dirname(__file__), "golden", "usp_kvcache_rear_u2.npz")
    spec, d = _load_usp(path)
    U, S_loc = spec["ulysses"], spec["s_loc"]
    n_patch, tok = 2, S_loc // 2
    B, S, H, D = d["k"].shape

    def image_order(x):
        # fixture rows are (rank, patch, i); the pipeline's image order is (patch, rank, i)
        return x.view(B, U, n_patch, tok, H, D).transpose(1, 2).reshape(B, S, H, D)

    order = opf.warmup_cache_order([U * tok] * n_patch, U)
    buf_k, buf_v = image_order(d["k"])[:, order].clone(), image_order(d["v"])[:, order].clone()
    assert torch.equal(buf_k, d["k"])               # after warm-up the buffer holds the gathered (rank-major) rows
    lo = U * tok                                    # image-order start of patch 1 = where the reference writes it
    buf_k[:, lo:lo + U * tok], buf_v[:, lo:lo + U * tok] = d["fresh_k"], d["fresh_v"]
    keys, vals = torch.cat([buf_k, d["jk"]], 1), torch.cat([buf_v, d["jv"]], 1)
    for r in range(U):
        q = torch.cat([d["fresh_q"][:, r * tok:(r + 1) * tok], d["jq"]], 1)      # "rear": [local; joint]
        torch.testing.assert_close(oa.sdpa(q, keys, vals), d[f"out_patch1_rank{r}"], rtol=2e-5, atol=2e-5)


# ----------------------------------------------------------------------------- attention processors
def _processor_case(name):
    golden = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
    with np.load(os.path.join(golden, "attn_processors.npz")) as f:
        spec = json.loads(str(f["spec"]))
        arrays = {k[len(name) + 1:]: torch.from_numpy(f[k]) for k in f.files if k.startswith(name + "/")}
    sd = {"a." + k: v for k, v in arrays.items() if not k.startswith(("in.", "out.")) and k not in ("cos", "sin")}
    rope = (arrays["cos"], arrays["sin"]) if "cos" in arrays else None
    return spec, sd, arrays, rope


def _close32(got, want):
    assert got.shape == want.shape
    assert (got - want).abs().max().item() <= 2e-5 * max(1.0, want.abs().max().item())


def test_oracle_attention_matches_the_reference_processors():
    """oracle/shaped_dit.py's attention of every block kind against what the reference's own attention processors
    return on the same weights and inputs (fixtures recorded by tests/golden/make_golden.py from the processors'
    __call__, CPU fp32): order of text and image rows, which rows are rotated, RMSNorm or LayerNorm QK norm."""
    from oracle import shaped_dit as osd
    # SD3: [image; text], no norm, no rotary table
    spec, sd, x, rope = _processor_case("joint_sd3")
    H, D = spec["heads"], spec["head_dim"]
    img, txt = osd.joint_attention(sd, "a", x["in.hidden"], x["in.encoder"], None, H, D, "rear")
    _close32(img, x["out.image"])
    _close32(txt, x["out.text"])
    # Flux double: [text; image], rotary rows for both
    spec, sd, x, rope = _processor_case("flux_double")
    img, txt = osd.joint_attention(sd, "a", x["in.hidden"], x["in.encoder"], rope, H, D, "front", rope_on_text=True)
    _close32(img, x["out.image"])
    _close32(txt, x["out.text"])
    # Flux single: the joint rows [text; image]; with and without the text / image split of the rotary rows
    spec, sd, x, rope = _processor_case("flux_single")
    _close32(osd.single_attention(sd, "a", x["in.hidden"], rope, H, D), x["out.joint"])
    _close32(osd.single_attention(sd, "a", x["in.hidden"], rope, H, D, text_len=spec["s_txt"]), x["out.joint"])
    # CogVideoX: [text; video], LayerNorm QK norm, rotary rows for the video only
    spec, sd, x, rope = _processor_case("cogvideox")
    joint = torch.cat([x["in.encoder"], x["in.hidden"]], dim=1)
    _close32(osd.cogvideox_attention(sd, "a", joint, spec["s_txt"], rope, H, D), x["out.joint"])
    # HunyuanVideo double: [video; text], rotary rows for the video only
    spec, sd, x, rope = _processor_case("hunyuan_double")
    img, txt = osd.joint_attention(sd, "a", x["in.hidden"], x["in.encoder"], rope, H, D, "rear", rope_on_text=False)
    _close32(torch.cat([img, txt], dim=1), x["out.joint"])
    # HunyuanVideo single: the processor concatenates [video; text] itself
    spec, sd, x, rope = _processor_case("hunyuan_single")
    joint = torch.cat([x["in.hidden"], x["in.encoder"]], dim=1)
    got = osd.single_attention(sd, "a", joint, rope, H, D, text_len=spec["s_txt"], text_first=False, rope_on_text=False)
    _close32(got, x["out.joint"])
