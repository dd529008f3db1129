"""Generates the golden fixtures in this directory from the reference's own source files.

Run it where the reference checkout is available:

    python tests/golden/make_golden.py --reference /path/to/Hetu-DiT

It never copies reference source into this repository: functions are lifted
from the reference files at run time (by AST for single functions, by loading
whole files under stub packages otherwise), executed on CPU, and only their
inputs and outputs are written out:

  bookkeeping.json   integer bookkeeping (patch metadata, rank groups, slice
                     ranges, migration plans, TP split table)
  rope.npz           apply_rotary_emb on seeded inputs
  usp_<case>.npz     hetuDiT*LongContextAttention / hetuDiTUlyssesAttention / ring attention / KV cache on
                     CPU `gloo` ranks, fp32 (--only usp, or --only usp:<name prefix> for some of them)
  attn_processors.npz  the attention processors' __call__ (SD3, Flux double / single, CogVideoX,
                     HunyuanVideo double / single) on a stand-in Attention module, fp32
                     (--only attn_processors)
  scheduler_step.npz the flow-matching Euler scheduler wrapper's step() per patch: new sample and when the
                     step index advances (--only scheduler_step)
  stage_split.json   which double / single blocks a pipeline stage keeps (_split_transformer_blocks)
                     (--only stage_split)
  stage_forward.npz  forward() of the SD3 and Flux transformer wrappers for every stage of 1- to 4-stage
                     pipelines on stand-in embedders / blocks / output layers, whole image and per patch
                     (--only stage_forward)
  pipefusion_order.json  per pipeline stage, the order of receives, receive-queue
                     operations, forwards, scheduler steps and sends that the SD3
                     pipeline's _sync_pipeline / _init_async_pipeline / _async_pipeline
                     produce with recording stand-ins (--only pipefusion_order)
  pos_embed_rows.json  which rows of the position table the patch-embedding wrapper
                     adds on every sequence-parallel rank, whole image and per
                     pipeline patch (--only pos_embed_rows)

The reference imports packages that are not installed here (diffusers, ray,
yunchang, flash_attn on CPU). Those imports are satisfied with stubs defined
below: yunchang's SeqAllToAll4D / RingComm / update_out_and_lse and flash-attn's
_flash_attn_forward are re-stated from their published behaviour with
torch.distributed (gloo) and fp32 torch math; everything else executed is the
reference's code.
"""
import argparse
import ast
import asyncio
import importlib.util
import json
import logging
import os
import sys
import types
from itertools import combinations

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


# ----------------------------------------------------------------------------- lifting helpers
def _find(tree, name, cls=None):
    body = tree.body
    if cls is not None:
        for node in body:
            if isinstance(node, ast.ClassDef) and node.name == cls:
                body = node.body
                break
        else:
            raise KeyError(cls)
    for node in body:
        if isinstance(node, (ast.FunctionDef, ast.AsyncFunctionDef, ast.ClassDef)) and node.name == name:
            return node
    raise KeyError(name)


def lift(path, name, cls=None, namespace=None):
    """Compile one function / class definition out of a reference file into `namespace`."""
    with open(path) as f:
        tree = ast.parse(f.read())
    node = _find(tree, name, cls)
    mod = ast.Module(body=[node], type_ignores=[])
    ns = dict(namespace or {})
    exec(compile(mod, path, "exec"), ns)
    return ns[name], ns


class _NS(types.SimpleNamespace):
    pass


# ----------------------------------------------------------------------------- bookkeeping
def gen_bookkeeping(ref):
    from typing import Any, Dict, List, Optional, Tuple, Union

    log = logging.getLogger("golden")
    out = {}

    # --- patch metadata --------------------------------------------------
    rs_path = os.path.join(ref, "hetu_dit/core/distributed/runtime_state.py")
    cases = []
    for variant, fname in (("image", "_calc_patches_metadata"), ("cogvideox", "_calc_cogvideox_patches_metadata")):
        for (h, w, vae, patch, npp, sp) in [
            (1024, 1024, 8, 2, 4, 1), (1024, 1024, 8, 2, 4, 2), (1024, 1024, 8, 2, 4, 4), (1024, 1024, 8, 2, 4, 8),
            (512, 512, 8, 2, 4, 1), (512, 512, 8, 2, 4, 2), (768, 768, 8, 2, 4, 1), (768, 768, 8, 2, 4, 2),
            (1536, 1536, 8, 2, 4, 1), (1536, 1536, 8, 2, 4, 2), (1536, 1536, 8, 2, 4, 4), (1024, 1024, 8, 2, 1, 1),
            (1024, 1024, 8, 2, 2, 2), (1024, 1024, 8, 2, 8, 1), (1024, 1024, 8, 2, 3, 1), (1024, 1024, 8, 2, 5, 2),
            (1024, 2048, 8, 2, 4, 2), (1152, 896, 8, 2, 4, 1), (1152, 896, 8, 2, 3, 2), (768, 1360, 8, 2, 1, 2),
            (768, 1360, 8, 2, 2, 4), (768, 1360, 8, 2, 4, 1), (1024, 1024, 16, 1, 4, 2), (720, 1280, 8, 2, 3, 1),
            (1000, 1000, 8, 2, 4, 1), (1080, 1920, 8, 2, 4, 1),
        ]:
            for rank in range(sp):
                ns = {
                    "get_sequence_parallel_world_size": lambda sp=sp: sp,
                    "get_sequence_parallel_rank": lambda rank=rank: rank,
                    "logger": log,
                }
                fn, _ = lift(rs_path, fname, cls="DiTRuntimeState", namespace=ns)
                self = _NS(
                    backbone_patch_size=patch, vae_scale_factor=vae, vae_scale_factor_spatial=vae,
                    vae_scale_factor_temporal=4,
                    input_config=_NS(height=h, width=w, num_frames=49),
                    parallel_config=_NS(pp_config=_NS(num_pipeline_patch=npp)),
                )
                rec = {"variant": variant, "height": h, "width": w, "vae": vae, "patch": patch,
                       "num_pipeline_patch": npp, "sp_world": sp, "sp_rank": rank}
                try:
                    fn(self)
                    rec["result"] = {k: getattr(self, k) for k in (
                        "num_pipeline_patch", "pp_patches_height", "pp_patches_start_idx_local",
                        "pp_patches_start_end_idx_global", "pp_patches_token_start_idx_local",
                        "pp_patches_token_start_end_idx_global", "pp_patches_token_num")}
                except ValueError as e:
                    rec["error"] = "ValueError"
                cases.append(rec)
    out["patches_metadata"] = cases

    # --- rank groups -------------------------------------------------------
    utils_ns = {}
    with open(os.path.join(ref, "hetu_dit/core/distributed/utils.py")) as f:
        exec(compile(f.read(), "utils.py", "exec"), utils_ns)
    RankGenerator = utils_ns["RankGenerator"]
    rg_cases = []
    for (tp, sp, pp, cfg, dp) in [(1, 8, 1, 1, 1), (1, 4, 2, 1, 1), (1, 2, 4, 1, 1), (2, 2, 2, 1, 1), (1, 2, 2, 2, 1),
                                  (1, 1, 4, 1, 2), (2, 1, 1, 1, 1), (1, 1, 1, 1, 1), (2, 2, 1, 2, 2), (1, 4, 1, 1, 2)]:
        for off in (0, 8):
            g = RankGenerator(tp, sp, pp, cfg, dp, "tp-sp-pp-cfg-dp", rank_offset=off)
            rg_cases.append({"tp": tp, "sp": sp, "pp": pp, "cfg": cfg, "dp": dp, "rank_offset": off,
                             "groups": {tok: g.get_ranks(tok) for tok in ("tp", "sp", "pp", "cfg", "dp", "tp-sp")}})
    out["rank_generator"] = rg_cases
    mo = utils_ns["generate_masked_orthogonal_rank_groups"]
    ddl_fn, _ = lift(os.path.join(ref, "hetu_dit/utils.py"), "estimate_ddl", namespace={})
    out["estimate_ddl"] = [{"t": {str(k): v for k, v in t.items()}, "ddl": ddl_fn(t)} for t in (
        {1: 0.144}, {1: 0.245, 4: 0.27}, {1: 0.45, 2: 0.37}, {1: 1.28, 4: 0.59}, {1: 1.28, 2: 0.75, 4: 0.59, 8: 0.5},
        {1: 10.0, 2: 5.5, 4: 3.0, 8: 2.2}, {1: 10.0, 2: 7.0}, {1: 100.0, 2: 51.0, 4: 26.0, 8: 20.0}, {1: 0.6, 8: 0.09})]
    # --- worker plan API: parameter lists of the methods the executor calls by name -----------------------------
    with open(os.path.join(ref, "hetu_dit/worker/worker.py")) as f:
        wtree = ast.parse(f.read())
    sigs = {}
    for node in ast.walk(wtree):
        if isinstance(node, ast.ClassDef) and node.name == "Worker":
            for fn in node.body:
                if isinstance(fn, (ast.FunctionDef, ast.AsyncFunctionDef)) and fn.name in (
                        "switch_parallel_env", "hotspa_model", "execute_diffusion_stage",
                        "execute_encode_diffusion_stage", "get_worker_state"):
                    sigs[fn.name] = {"params": [a.arg for a in fn.args.args if a.arg != "self"],
                                     "coroutine": isinstance(fn, ast.AsyncFunctionDef)}
    out["worker_signatures"] = sigs
    # --- the status record the engine polls: get_worker_state run on stand-in workers with a fixed clock ---------
    clock = _NS(perf_counter=lambda: 1000.0)
    state_fn, _ = lift(os.path.join(ref, "hetu_dit/worker/worker.py"), "get_worker_state", cls="Worker",
                       namespace={"time": clock, "torch": _NS(cuda=_NS(memory_allocated=lambda: 0))})
    out["worker_state"] = []
    for states in ({}, {"running_task": "t1", "task_start_time": 990.0},
                   {"running_task": "t2", "task_start_time": 990.0, "stage_name": "diffusion",
                    "diffusion_start_time": 995.5, "estimated_running_time": 25.0},
                   {"running_task": "t3", "task_start_time": 990.0, "stage_name": "diffusion",
                    "diffusion_start_time": 995.5, "estimated_running_time": 4.0},
                   {"running_task": "t4", "task_start_time": 990.0, "stage_name": "vae", "estimated_running_time": 10.0},
                   {"stage_name": "diffusion", "diffusion_start_time": 1000.0, "estimated_running_time": 3.0}):
        out["worker_state"].append({"now": 1000.0, "rank": 3, "states": states,
                                    "result": state_fn(_NS(rank=3, states=dict(states)))})
    # --- operator / coordinator / cache surface: parameter names and literal defaults, as written in the source --
    def surface(rel, wanted):
        with open(os.path.join(ref, rel)) as f:
            t = ast.parse(f.read())
        got = {}
        for node in ast.walk(t):
            if isinstance(node, ast.ClassDef) and node.name in wanted:
                for fn in node.body:
                    if isinstance(fn, (ast.FunctionDef, ast.AsyncFunctionDef)) and fn.name in wanted[node.name]:
                        args = [a.arg for a in fn.args.args if a.arg != "self"]
                        defaults = {}
                        for a, d in zip(args[len(args) - len(fn.args.defaults):], fn.args.defaults):
                            try:
                                defaults[a] = ast.literal_eval(d)
                            except ValueError:
                                defaults[a] = "<expression>"
                        kwonly = [a.arg for a in fn.args.kwonlyargs]
                        for a, d in zip(kwonly, fn.args.kw_defaults):
                            if d is not None:
                                try:
                                    defaults[a] = ast.literal_eval(d)
                                except ValueError:
                                    defaults[a] = "<expression>"
                        got[f"{node.name}.{fn.name}"] = {"params": args + kwonly, "defaults": defaults,
                                                         "coroutine": isinstance(fn, ast.AsyncFunctionDef)}
        return got
    api = {}
    api.update(surface("hetu_dit/core/parallel/hybrid/attn_layer.py", {
        "hetuDiTLongContextAttention": ["__init__", "forward"], "hetuDiTFluxLongContextAttention": ["__init__", "forward"],
        "hetuDiTJointLongContextAttention": ["__init__", "forward"]}))
    api.update(surface("hetu_dit/core/parallel/ulysses/attn_layer.py", {"hetuDiTUlyssesAttention": ["__init__", "forward"]}))
    api.update(surface("hetu_dit/core/distributed/group_coordinator.py", {"PipelineGroupCoordinator": [
        "pipeline_send", "pipeline_isend", "pipeline_recv", "add_pipeline_recv_task", "recv_next",
        "get_pipeline_recv_data", "reset_buffer"]}))
    api.update(surface("hetu_dit/core/resource_manager/cache_manager.py", {"CacheManager": [
        "update_and_get_kv_cache", "register_cache_entry"]}))
    api.update(surface("hetu_dit/model_executor/cache/base_cache.py", {"BaseBlockCache": ["adjust_pipeline"]}))
    api.update(surface("hetu_dit/core/distributed/runtime_state.py", {"DiTRuntimeState": [
        "set_input_parameters", "set_video_input_parameters", "set_patched_mode", "next_patch"]}))
    api.update(surface("hetu_dit/core/distributed/group_coordinator.py", {"GroupCoordinator": ["all_gather"],
                                                                          "PipelineGroupCoordinator": ["set_config"]}))
    # module-level: the ring attention entry point
    with open(os.path.join(ref, "hetu_dit/core/parallel/ring/ring_flash_attn.py")) as f:
        fn = _find(ast.parse(f.read()), "ring_flash_attn_func")
    names = [a.arg for a in fn.args.args]
    api["ring_flash_attn_func"] = {"params": names, "coroutine": False, "defaults": {
        a: ast.literal_eval(d) for a, d in zip(names[len(names) - len(fn.args.defaults):], fn.args.defaults)}}
    out["api_surface"] = api
    out["masked_orthogonal"] = [
        {"world": 24, "sizes": [2, 3, 4], "mask": m, "groups": mo(24, [2, 3, 4], m)}
        for m in ([False, True, False], [True, False, True], [True, True, True], [False, False, False])
    ]

    ps_path = os.path.join(ref, "hetu_dit/core/distributed/parallel_state.py")
    fake_torch = _NS(distributed=_NS(new_group=lambda ranks, backend=None: list(ranks)))
    sp_fn, _ = lift(ps_path, "set_seq_parallel_pg", namespace={"torch": fake_torch, "List": List})
    sp_cases = []
    for (u, r, ranks) in [(4, 2, list(range(8))), (2, 4, list(range(8))), (8, 1, list(range(8))), (1, 8, list(range(8))),
                          (2, 2, [0, 3, 4, 7]), (2, 1, [5, 2]), (1, 2, [1, 6]), (2, 2, list(range(8))),
                          (1, 1, [3]), (4, 1, [7, 1, 3, 5])]:
        for low in (True, False):
            world = len(ranks)
            per_rank = {}
            for rank in sorted(ranks):
                upg, rpg = sp_fn(u, r, rank, world, ranks, use_ulysses_low=low)
                per_rank[str(rank)] = {"ulysses": upg, "ring": rpg}
            sp_cases.append({"ulysses": u, "ring": r, "ranks": ranks, "use_ulysses_low": low, "per_rank": per_rank})
    out["seq_parallel_groups"] = sp_cases

    pg_ns = {"combinations": combinations, "np": np, "List": List}
    comb_fn, _ = lift(ps_path, "_generate_rank_combinations", cls="ParallelGroups", namespace=pg_ns)
    part_fn, _ = lift(ps_path, "_generate_group_ranks", cls="ParallelGroups", namespace=pg_ns)
    me = _NS(valid_degrees=[1, 2, 4, 8])
    out["rank_combinations"] = [{"world": w, "base": b, "result": comb_fn(me, w, b)} for w, b in ((4, 0), (8, 0), (2, 8))]
    out["group_partitions"] = [{"ranks": rk, "result": part_fn(me, rk)}
                               for rk in ([0], [0, 1], [0, 1, 2, 3], [1, 3, 5, 7], list(range(8)))]

    # --- slice ranges --------------------------------------------------------
    u_path = os.path.join(ref, "hetu_dit/utils.py")
    r2i_round, _ = lift(u_path, "range_to_indices")
    meta_fn, _ = lift(u_path, "get_gpu_metadata")
    bc_path = os.path.join(ref, "hetu_dit/model_executor/cache/base_cache.py")
    r2i_trunc, _ = lift(bc_path, "range_to_indices", cls="BaseBlockCache", namespace={"Tuple": Tuple, "logger": log})
    ranges = []
    for world in (1, 2, 3, 4, 8):
        for rank in range(world):
            ranges.append((rank / world, rank / world + 1.0 / world))
            ranges.append((rank * (1.0 / world), rank * (1.0 / world) + 1.0 / world))
    ranges += [(0.0, 1.0), (0.25, 0.75), (0.5, 0.5), (0.9, 0.3), (0.0, 0.3333), (0.3333, 0.6666), (0.6666, 1.0)]
    r2i = []
    for rng in ranges:
        for total in (0, 1, 7, 24, 38, 57, 1536, 3072, 4096, 6144, 12288, 18432, 333, 1000):
            r2i.append({"range": list(rng), "total": total, "round": list(r2i_round(rng, total)),
                        "trunc": list(r2i_trunc(None, rng, total))})
    out["range_to_indices"] = r2i
    out["gpu_metadata"] = [
        {"pp_rank": pr, "pp_world": pw, "tp_rank": tr, "tp_world": tw,
         "result": {k: list(v) for k, v in meta_fn(pr, pw, tr, tw).items()}}
        for pw in (1, 2, 3, 4, 8) for pr in range(pw) for tw in (1, 2, 3, 4, 8) for tr in range(tw)
    ]

    # --- TP split table ------------------------------------------------------
    tc_path = os.path.join(ref, "hetu_dit/model_executor/cache/transformer_cache.py")
    choose_fn, _ = lift(tc_path, "choose_tp_split_type", cls="TransformerBlockCache", namespace={"Optional": Optional})
    det_fn, _ = lift(tc_path, "determine_tp_split_type_by_name", cls="TransformerBlockCache")
    tself = _NS()
    tself.determine_tp_split_type_by_name = lambda n: det_fn(tself, n)
    names = [f"{a}.module.{n}" for a in ("attn", "attn1", "attn2") for n in
             ("to_q", "to_k", "to_v", "add_k_proj", "add_q_proj", "add_v_proj", "to_add_out", "to_out.0", "to_out.1",
              "norm_q")]
    names += ["ff.module.net.0.proj", "ff.module.net.2", "ff_context.module.net.0.proj", "ff_context.module.net.2",
              "ff.module.net.0", "norm1.linear", "proj_mlp", "proj_out", "attn.to_q", "ff.net.2"]
    out["tp_split_type"] = [{"name": n, "result": choose_fn(tself, n)} for n in names]

    # --- migration plans -------------------------------------------------------
    import torch.nn as nn
    from dataclasses import dataclass, field
    dc_ns = {"dataclass": dataclass, "field": field, "Optional": Optional, "Tuple": Tuple, "List": List, "nn": nn}
    NeededPiece, dc_ns2 = lift(bc_path, "NeededPiece", namespace=dc_ns)
    dc_ns2.pop("__builtins__", None)
    Plan, _ = lift(bc_path, "DataReconstructionPlan", namespace={**dc_ns, "NeededPiece": NeededPiece})

    class Stop(Exception):
        pass

    class FakeLinearBlock(nn.Module):
        """A block whose named_modules() yields Linear layers under the names the reference adjusts."""

        def __init__(self, spec):
            super().__init__()
            for path, out_f, in_f, bias in spec:
                parts = path.split(".")
                mod = self
                for p in parts[:-1]:
                    if not hasattr(mod, p):
                        mod.add_module(p, nn.Module())
                    mod = getattr(mod, p)
                with torch.device("meta"):
                    mod.add_module(parts[-1], nn.Linear(in_f, out_f, bias=bias))

    def block_spec(kind, dm):
        if kind == "sd3":
            return [("attn.module.to_q", dm, dm, True), ("attn.module.to_k", dm, dm, True),
                    ("attn.module.to_v", dm, dm, True), ("attn.module.add_k_proj", dm, dm, True),
                    ("attn.module.add_v_proj", dm, dm, True), ("attn.module.add_q_proj", dm, dm, True),
                    ("attn.module.to_out.0", dm, dm, True), ("attn.module.to_add_out", dm, dm, True),
                    ("ff.module.net.0.proj", 4 * dm, dm, True), ("ff.module.net.2", dm, 4 * dm, True),
                    ("ff_context.module.net.0.proj", 4 * dm, dm, True), ("ff_context.module.net.2", dm, 4 * dm, True),
                    ("norm1.linear", 6 * dm, dm, True)]
        return [("attn.module.to_q", dm, dm, True), ("attn.module.to_k", dm, dm, False),
                ("attn.module.to_v", dm, dm, True), ("attn.module.to_out.0", dm, dm, True),
                ("proj_mlp", 4 * dm, dm, True)]

    adj_fn, _ = lift(bc_path, "_adjust_pipeline_legacy", cls="BaseBlockCache", namespace={
        "nn": nn, "Optional": Optional, "Dict": Dict, "List": List, "Tuple": Tuple, "logger": log,
        "get_runtime_state": lambda: _NS(runtime_config=_NS(adjust_strategy="cache")),
        "DataReconstructionPlan": Plan, "NeededPiece": NeededPiece,
    })

    plan_cases = []
    for (kind, dm, nblocks, old_pp, new_pp, cached, target, slice_bias) in [
        ("sd3", 1536, 4, (0.0, 1.0), (0.0, 1.0), {0: (0.0, 0.5), 1: (0.0, 0.5), 2: (0.0, 0.5), 3: (0.0, 0.5)}, (0.0, 1.0), True),
        ("sd3", 1536, 4, (0.0, 1.0), (0.0, 1.0), {0: (0.0, 1.0), 1: (0.0, 1.0), 2: (0.0, 1.0), 3: (0.0, 1.0)}, (0.5, 1.0), True),
        ("sd3", 1536, 4, (0.0, 0.5), (0.5, 1.0), {0: (0.0, 1.0), 1: (0.0, 1.0)}, (0.0, 1.0), True),
        ("sd3", 1536, 8, (0.0, 0.5), (0.25, 0.75), {0: (0.0, 0.5), 1: (0.0, 0.5), 2: (0.25, 0.5), 3: (0.0, 0.25)}, (0.25, 0.75), True),
        ("flux1", 3072, 6, (0.0, 1.0), (0.0, 1.0), {i: (0.25, 0.5) for i in range(6)}, (0.0, 1.0), True),
        ("flux1", 3072, 6, (0.0, 1.0), (0.0, 1.0), {i: (0.25, 0.5) for i in range(6)}, (0.0, 1.0), False),
        ("flux1", 3072, 3, (0.0, 1.0), (0.0, 1.0), {0: (0.0, 1.0 / 3), 2: (2.0 / 3, 1.0)}, (1.0 / 3, 1.0), True),
        ("sd3", 1000, 3, (0.0, 1.0), (0.0, 1.0), {0: (0.0, 1.0 / 3), 1: (1.0 / 3, 1.0 / 3 + 1.0 / 3)}, (0.0, 0.5), True),
    ]:
        cpu_blocks = [FakeLinearBlock(block_spec(kind, dm)) for _ in range(nblocks)]

        class FakeSelf:
            def __init__(self):
                self.cache = {i: (None, tuple(r)) for i, r in cached.items()}
                self.active_block_indices = sorted(cached.keys())

            def range_to_indices(self, rng, total):
                return r2i_trunc(self, rng, total)

            def get_total_blocks(self, m):
                return nblocks

            def get_cpu_block_for_index(self, m, idx):
                return cpu_blocks[idx]

            def choose_tp_split_type(self, name):
                return choose_fn(tself, name)

            def __getattr__(self, name):
                raise Stop(name)

        fs = FakeSelf()
        old_tp = next(iter(cached.values())) if cached else (0.0, 1.0)
        try:
            asyncio.run(adj_fn(fs, None, None, old_pp, new_pp, old_tp, target, slice_bias, None))
        except Stop:
            pass
        pieces = [{k: getattr(p, k) for k in ("uid", "block_index", "layer_path", "tensor_type", "split_dim", "full_size",
                                              "abs_start_idx", "abs_end_idx", "dest_offset")}
                  for p in fs.__dict__.get("_last_p2p_all_pieces", [])]
        plan_cases.append({
            "kind": kind, "hidden": dm, "num_blocks": nblocks, "new_pp": list(new_pp),
            "cached": {str(k): list(v) for k, v in cached.items()}, "target_tp": list(target), "slice_bias": slice_bias,
            "linears": [[n, o, i, b] for n, o, i, b in block_spec(kind, dm)], "pieces": pieces,
        })
    out["migration_plans"] = plan_cases

    with open(os.path.join(HERE, "bookkeeping.json"), "w") as f:
        json.dump(out, f, separators=(",", ":"))
    print("bookkeeping.json:", {k: len(v) for k, v in out.items()})


# ----------------------------------------------------------------------------- RoPE
def gen_rope(ref):
    from typing import Tuple, Union
    path = os.path.join(ref, "hetu_dit/model_executor/diffusion_executor/layers/attention_processor.py")
    fn, _ = lift(path, "apply_rotary_emb", namespace={"torch": torch, "Union": Union, "Tuple": Tuple})
    g = torch.Generator().manual_seed(1234)
    data = {}
    for i, (B, H, S, D) in enumerate([(1, 2, 37, 64), (2, 3, 16, 128)]):
        x = torch.randn(B, H, S, D, generator=g)
        ang = torch.rand(S, D // 2, generator=g) * 6.28
        cos = torch.cos(ang).repeat_interleave(2, dim=-1)
        sin = torch.sin(ang).repeat_interleave(2, dim=-1)
        data[f"x{i}"] = x.numpy()
        data[f"cos{i}"] = cos.numpy()
        data[f"sin{i}"] = sin.numpy()
        data[f"y{i}"] = fn(x, (cos, sin)).numpy()
        xb = x.to(torch.bfloat16)
        data[f"yb{i}"] = fn(xb, (cos, sin)).float().numpy()
    np.savez_compressed(os.path.join(HERE, "rope.npz"), **data)
    print("rope.npz written")


# ----------------------------------------------------------------------------- USP attention on gloo ranks
def _install_stub_packages(ref, state):
    """Registers stub third-party modules and loads the reference's attention files under their real names."""
    import torch.distributed as dist

    def pkg(name):
        m = types.ModuleType(name)
        m.__path__ = []
        sys.modules[name] = m
        return m

    def load(name, relpath):
        spec = importlib.util.spec_from_file_location(name, os.path.join(ref, relpath))
        m = importlib.util.module_from_spec(spec)
        sys.modules[name] = m
        spec.loader.exec_module(m)
        parent, _, leaf = name.rpartition(".")
        setattr(sys.modules[parent], leaf, m)
        return m

    # ---- hetu_dit stubs ---------------------------------------------------
    for n in ("hetu_dit", "hetu_dit.core", "hetu_dit.core.distributed", "hetu_dit.core.resource_manager",
              "hetu_dit.core.parallel", "hetu_dit.core.parallel.hybrid", "hetu_dit.core.parallel.ring",
              "hetu_dit.core.parallel.ulysses"):
        pkg(n)
    lg = types.ModuleType("hetu_dit.logger")
    lg.init_logger = lambda name: logging.getLogger(name)
    sys.modules["hetu_dit.logger"] = lg
    ps = types.ModuleType("hetu_dit.core.distributed.parallel_state")
    ps.get_sequence_parallel_world_size = lambda: state.sp_world
    sys.modules["hetu_dit.core.distributed.parallel_state"] = ps
    rs = types.ModuleType("hetu_dit.core.distributed.runtime_state")
    rs.runtime_state_is_initialized = lambda: state.runtime is not None
    rs.get_runtime_state = lambda: state.runtime
    sys.modules["hetu_dit.core.distributed.runtime_state"] = rs
    d = sys.modules["hetu_dit.core.distributed"]
    d.get_ulysses_parallel_world_size = lambda: state.ulysses
    d.get_runtime_state = lambda: state.runtime
    d.runtime_state = rs
    d.parallel_state = ps

    # ---- yunchang 0.3.5 stubs (published behaviour, gloo transport) ---------
    class _PG:
        ULYSSES_PG = None
        RING_PG = None

    class SeqAllToAll4D:
        @staticmethod
        def apply(group, x, scatter_idx, gather_idx):
            world = dist.get_world_size(group)
            if world == 1:
                return x
            rank = dist.get_rank(group)
            gathered = [torch.empty_like(x) for _ in range(world)]
            dist.all_gather(gathered, x.contiguous(), group=group)
            parts = [torch.chunk(g, world, dim=scatter_idx)[rank] for g in gathered]
            return torch.cat(parts, dim=gather_idx).contiguous()

    class RingComm:
        def __init__(self, process_group):
            self._pg = process_group
            self.rank = dist.get_rank(process_group)
            self.world_size = dist.get_world_size(process_group)
            self._ops, self._reqs = [], None
            ranks = dist.get_process_group_ranks(process_group)
            self.send_rank = ranks[(self.rank + 1) % self.world_size]
            self.recv_rank = ranks[(self.rank - 1) % self.world_size]

        def send_recv(self, to_send, recv_tensor=None):
            res = torch.empty_like(to_send) if recv_tensor is None else recv_tensor
            self._ops.append(dist.P2POp(dist.isend, to_send.contiguous(), self.send_rank, group=self._pg))
            self._ops.append(dist.P2POp(dist.irecv, res, self.recv_rank, group=self._pg))
            return res

        def commit(self):
            self._reqs = dist.batch_isend_irecv(self._ops)

        def wait(self):
            for r in self._reqs:
                r.wait()
            self._reqs, self._ops = None, []

    def update_out_and_lse(out, lse, block_out, block_lse, slice_=None):
        block_out = block_out.to(torch.float32)
        block_lse = block_lse.transpose(-2, -1).unsqueeze(dim=-1)
        if out is None:
            return block_out, block_lse
        new_lse = lse + torch.log(1 + torch.exp(block_lse - lse))
        out = torch.exp(lse - new_lse) * out + torch.exp(block_lse - new_lse) * block_out
        return out, new_lse

    class LongContextAttention(torch.nn.Module):
        def __init__(self, scatter_idx=2, gather_idx=1, ring_impl_type="basic", use_pack_qkv=False, **kw):
            super().__init__()
            self.scatter_idx, self.gather_idx = scatter_idx, gather_idx
            self.ring_impl_type, self.use_pack_qkv = ring_impl_type, use_pack_qkv

    class UlyssesAttention(torch.nn.Module):
        pass

    class RingFlashAttnFunc(torch.autograd.Function):
        pass

    def torch_attn(q, k, v, dropout_p=0.0, softmax_scale=None, causal=False, *args, **kwargs):
        o = torch.nn.functional.scaled_dot_product_attention(
            q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), dropout_p=0.0, is_causal=False, scale=softmax_scale)
        return o.transpose(1, 2)

    y = pkg("yunchang")
    y.LongContextAttention, y.UlyssesAttention = LongContextAttention, UlyssesAttention
    pkg("yunchang.comm")
    m = types.ModuleType("yunchang.comm.all_to_all"); m.SeqAllToAll4D = SeqAllToAll4D
    sys.modules[m.__name__] = m
    m = types.ModuleType("yunchang.globals"); m.PROCESS_GROUP = _PG
    sys.modules[m.__name__] = m
    r = pkg("yunchang.ring")
    r.zigzag_ring_flash_attn_func = r.stripe_flash_attn_func = None
    m = types.ModuleType("yunchang.ring.utils"); m.RingComm, m.update_out_and_lse = RingComm, update_out_and_lse
    sys.modules[m.__name__] = m
    m = types.ModuleType("yunchang.ring.ring_flash_attn"); m.RingFlashAttnFunc = RingFlashAttnFunc
    sys.modules[m.__name__] = m
    pkg("yunchang.ulysses")
    m = types.ModuleType("yunchang.ulysses.attn_layer"); m.torch_attn = torch_attn
    sys.modules[m.__name__] = m

    # ---- flash-attn stub: exact fp32 attention, 8-tuple like flash-attn 2.6 -------
    def _flash_attn_forward(q, k, v, dropout_p, softmax_scale, causal, window_size, softcap, alibi_slopes, return_softmax):
        assert not causal and dropout_p == 0
        s = torch.einsum("bqhd,bkhd->bhqk", q.float(), k.float()) * softmax_scale
        lse = torch.logsumexp(s, dim=-1)
        out = torch.einsum("bhqk,bkhd->bqhd", torch.exp(s - lse.unsqueeze(-1)), v.float()).to(q.dtype)
        return out, q, k, v, out, lse, None, None

    fa = pkg("flash_attn")
    m = types.ModuleType("flash_attn.flash_attn_interface"); m._flash_attn_forward = _flash_attn_forward
    sys.modules[m.__name__] = m
    fa.flash_attn_interface = m

    # ---- the reference's own files ----------------------------------------------
    cm = load("hetu_dit.core.resource_manager.cache_manager", "hetu_dit/core/resource_manager/cache_manager.py")
    ring = load("hetu_dit.core.parallel.ring.ring_flash_attn", "hetu_dit/core/parallel/ring/ring_flash_attn.py")
    sys.modules["hetu_dit.core.parallel.ring"].ring_flash_attn_func = ring.ring_flash_attn_func
    load("hetu_dit.core.parallel.hybrid.utils", "hetu_dit/core/parallel/hybrid/utils.py")
    hyb = load("hetu_dit.core.parallel.hybrid.attn_layer", "hetu_dit/core/parallel/hybrid/attn_layer.py")
    # the Ulysses-only operator asks for the GPU's name when it is built (to rule out flash-attn on old parts)
    torch.cuda.get_device_name = lambda *a, **k: "stand-in"
    uly = load("hetu_dit.core.parallel.ulysses.attn_layer", "hetu_dit/core/parallel/ulysses/attn_layer.py")
    hyb.hetuDiTUlyssesAttention = uly.hetuDiTUlyssesAttention
    return _PG, cm, ring, hyb


USP_CASES = {
    # name: (world, ulysses, ring, class, joint_strategy, S_loc, S_txt, H, D, kv_cache)
    "plain_u2": (2, 2, 1, "hetuDiTLongContextAttention", "none", 40, 0, 4, 64, False),
    "flux_front_u2": (2, 2, 1, "hetuDiTFluxLongContextAttention", "front", 40, 24, 4, 64, False),
    "joint_rear_u2r2": (4, 2, 2, "hetuDiTJointLongContextAttention", "rear", 24, 13, 4, 64, False),
    "joint_front_r2": (2, 1, 2, "hetuDiTJointLongContextAttention", "front", 33, 9, 2, 128, False),
    "joint_rear_u4": (4, 4, 1, "hetuDiTJointLongContextAttention", "rear", 16, 7, 8, 64, False),
    "joint_rear_r4": (4, 1, 4, "hetuDiTJointLongContextAttention", "rear", 20, 5, 2, 64, False),
    "kvcache_rear_u2": (2, 2, 1, "hetuDiTJointLongContextAttention", "rear", 32, 11, 4, 64, True),
    # the Ulysses-only operator (ulysses/attn_layer.py), built the way the processors build it without flash-attn
    "ulysses_plain_u2": (2, 2, 1, "hetuDiTUlyssesAttention", "none", 40, 0, 4, 64, False,
                         {"use_fa": False, "use_kv_cache": False}),
    "ulysses_rear_u2": (2, 2, 1, "hetuDiTUlyssesAttention", "rear", 36, 10, 4, 128, False,
                        {"use_fa": False, "use_kv_cache": False}),
    "ulysses_kvcache_front_u2": (2, 2, 1, "hetuDiTUlyssesAttention", "front", 32, 9, 4, 64, True,
                                 {"use_fa": False, "use_kv_cache": True}),
}


def _usp_worker(rank, world, ref, name, port, outdir):
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    _, U, R, cls_name, strategy, S_loc, S_txt, H, D, kv_cache = USP_CASES[name][:10]
    init_kw = USP_CASES[name][10] if len(USP_CASES[name]) > 10 else {}
    state = _NS(sp_world=U * R, ulysses=U, runtime=None)
    PG, cm, ring_mod, hyb = _install_stub_packages(ref, state)
    # Ulysses groups: consecutive ranks; ring groups: stride U (parallel_state.py:679-712).
    for i in range(R):
        g = dist.new_group(list(range(i * U, (i + 1) * U)), backend="gloo")
        if rank // U == i:
            PG.ULYSSES_PG = g
    for i in range(U):
        g = dist.new_group(list(range(i, U * R, U)), backend="gloo")
        if rank % U == i:
            PG.RING_PG = g

    gen = torch.Generator().manual_seed(1000 + sum(map(ord, name)))
    B = 1
    P = U * R
    full = {k: torch.randn(B, S_loc * P, H, D, generator=gen) for k in ("q", "k", "v")}
    joint = {k: torch.randn(B, S_txt, H, D, generator=gen) for k in ("jq", "jk", "jv")} if S_txt else {}
    sl = slice(rank * S_loc, (rank + 1) * S_loc)
    q, k, v = (full[n][:, sl].contiguous() for n in ("q", "k", "v"))
    layer = getattr(hyb, cls_name)(**init_kw)
    kwargs = {}
    if strategy != "none":
        kwargs = dict(joint_tensor_query=joint["jq"], joint_tensor_key=joint["jk"], joint_tensor_value=joint["jv"],
                      joint_strategy=strategy)
    save = {}
    if not kv_cache:
        out = layer(None, q, k, v, **kwargs)
        save["out"] = out.numpy()
    else:
        # PipeFusion + SP: a warm-up (whole image) call fills the stale-KV buffer, then one patch call reuses it.
        n_patch = 2
        tok = S_loc // n_patch
        rt = _NS(num_pipeline_patch=n_patch, patch_mode=False, pipeline_patch_idx=0,
                 pp_patches_token_num=[tok] * n_patch,
                 pp_patches_token_start_idx_local=[i * tok for i in range(n_patch + 1)])
        state.runtime = rt
        attn_obj = object()
        cm.get_cache_manager().register_cache_entry(attn_obj, "attn", "sequence_parallel_attn_cache")
        out0 = layer(attn_obj, q, k, v, **kwargs)
        save["out_warmup"] = out0.numpy()
        # new activations for patch 1 only
        fresh = {n: torch.randn(B, tok * P, H, D, generator=gen) for n in ("q", "k", "v")}
        psl = slice(rank * tok, (rank + 1) * tok)
        rt.patch_mode, rt.pipeline_patch_idx = True, 1
        out1 = layer(attn_obj, fresh["q"][:, psl].contiguous(), fresh["k"][:, psl].contiguous(),
                     fresh["v"][:, psl].contiguous(), **kwargs)
        save["out_patch1"] = out1.numpy()
        if rank == 0:
            for n in ("q", "k", "v"):
                save[f"fresh_{n}"] = fresh[n].numpy()
    np.savez_compressed(os.path.join(outdir, f"rank{rank}.npz"), **save)
    if rank == 0:
        inputs = {n: t.numpy() for n, t in {**full, **joint}.items()}
        np.savez_compressed(os.path.join(outdir, "inputs.npz"), **inputs)
    dist.barrier()
    dist.destroy_process_group()


def gen_usp(ref, only=None):
    import tempfile
    import torch.multiprocessing as mp
    port = 29611
    for name, spec in USP_CASES.items():
        if only and not name.startswith(only):
            continue
        world = spec[0]
        with tempfile.TemporaryDirectory() as tmp:
            mp.spawn(_usp_worker, args=(world, ref, name, port, tmp), nprocs=world, join=True)
            port += 1
            merged = {}
            with np.load(os.path.join(tmp, "inputs.npz")) as f:
                merged.update({k: f[k] for k in f.files})
            for r in range(world):
                with np.load(os.path.join(tmp, f"rank{r}.npz")) as f:
                    for k in f.files:
                        merged[k if k.startswith("fresh_") else f"{k}_rank{r}"] = f[k]
            merged["spec"] = np.array(json.dumps({
                "world": world, "ulysses": spec[1], "ring": spec[2], "cls": spec[3], "joint_strategy": spec[4],
                "s_loc": spec[5], "s_txt": spec[6], "heads": spec[7], "head_dim": spec[8], "kv_cache": spec[9]}))
            np.savez_compressed(os.path.join(HERE, f"usp_{name}.npz"), **merged)
            print(f"usp_{name}.npz written")


# ----------------------------------------------------------------------------- PipeFusion schedule order
PIPEFUSION_CASES = [
    # (pipeline stages, patches, denoising steps, warm-up steps)
    (2, 2, 3, 1), (2, 4, 4, 1), (2, 4, 3, 0), (3, 3, 4, 1), (4, 4, 3, 1), (4, 8, 4, 2), (2, 4, 2, 2), (1, 1, 3, 1),
    (4, 2, 3, 1),
]


def _lift_method_undecorated(path, name, cls, namespace):
    with open(path) as f:
        tree = ast.parse(f.read())
    node = _find(tree, name, cls)
    node.decorator_list = []
    ns = dict(namespace)
    exec(compile(ast.Module(body=[node], type_ignores=[]), path, "exec"), ns)
    return ns[name]


def gen_pipefusion_order(ref):
    """Runs the reference's _sync_pipeline / _init_async_pipeline / _async_pipeline of the SD3 pipeline
    (model_executor/pipelines/pipeline_stable_diffusion_3.py:1352-1678) and of the Flux pipeline
    (pipelines/pipeline_flux.py:428-760) for every stage of a few pipeline shapes with a recording stand-in for the
    pipeline group, the backbone and the scheduler, and writes per stage the order of receives, queue operations,
    forwards, scheduler steps and sends."""
    from typing import Callable, Dict, List, Optional
    families = {
        "sd3": ("hetu_dit/model_executor/pipelines/pipeline_stable_diffusion_3.py", "hetuDiTStableDiffusion3Pipeline"),
        "flux": ("hetu_dit/model_executor/pipelines/pipeline_flux.py", "hetuDiTFluxPipeline"),
    }
    cases = []
    for family, (rel, cls) in families.items():
        path = os.path.join(ref, rel)
        for (stages, n_patch, n_steps, warmup) in PIPEFUSION_CASES:
            for stage in range(stages):
                events = []
                patch_h = 2      # SD3: latent rows per patch; Flux: tokens per patch
                flux = family == "flux"

                def whole():
                    return torch.zeros(1, patch_h * n_patch, 4) if flux else torch.zeros(1, 4, patch_h * n_patch, 4)

                def one_patch():
                    return torch.zeros(1, patch_h, 4) if flux else torch.zeros(1, 4, patch_h, 4)

                class Group:
                    def pipeline_recv(self, idx=-1, name="latent"):
                        events.append(["recv", name or "latent", idx])
                        return whole() if (name or "latent") == "latent" else "text"

                    def pipeline_send(self, tensor, name="latent", segment_idx=-1):
                        events.append(["send", name, segment_idx])

                    pipeline_isend = pipeline_send

                    def add_pipeline_recv_task(self, idx=-1, name="latent"):
                        events.append(["add_recv_task", name or "latent", idx])

                    def recv_next(self):
                        events.append(["recv_next"])

                    def get_pipeline_recv_data(self, idx=-1, name="latent"):
                        events.append(["get", name, idx])
                        return one_patch() if name == "latent" else "text"

                class State:
                    num_pipeline_patch = n_patch
                    pp_patches_height = [patch_h] * n_patch
                    pp_patches_token_num = [patch_h] * n_patch
                    pp_patches_start_idx_local = [patch_h * i for i in range(n_patch + 1)]
                    pp_patches_token_start_idx_local = [patch_h * i for i in range(n_patch + 1)]
                    pp_patches_token_start_end_idx_global = [(patch_h * i, patch_h * (i + 1)) for i in range(n_patch)]
                    runtime_config = _NS(warmup_steps=warmup)
                    pipeline_patch_idx = 0

                    def set_patched_mode(self, patch_mode):
                        events.append(["patched_mode", bool(patch_mode)])
                        self.pipeline_patch_idx = 0

                    def next_patch(self):
                        self.pipeline_patch_idx = (self.pipeline_patch_idx + 1) % n_patch

                state, group = State(), Group()
                prompt = "prompt"

                class Pipe:
                    interrupt = False
                    scheduler = _NS(order=1)

                    def _backbone_forward(self, latents, encoder_hidden_states, pooled_prompt_embeds, t, **_):
                        events.append(["forward", state.pipeline_patch_idx, int(t),
                                       "prompt" if encoder_hidden_states is prompt else "received"])
                        return latents, "text"

                    def _scheduler_step(self, noise_pred, last, t):
                        events.append(["step", int(t)])
                        return noise_pred

                if flux:
                    def _init_sync(self, latents, latent_image_ids):
                        events.append(["patched_mode", False])  # what the reference's _init_sync_pipeline does first
                        state.pipeline_patch_idx = 0
                        return latents, latent_image_ids
                else:
                    def _init_sync(self, latents):
                        events.append(["patched_mode", False])
                        state.pipeline_patch_idx = 0
                        return latents
                Pipe._init_sync_pipeline = _init_sync

                ns = {
                    "torch": torch, "List": List, "Optional": Optional, "Callable": Callable, "Dict": Dict,
                    "logger": logging.getLogger("golden"), "XLA_AVAILABLE": False,
                    "get_runtime_state": lambda: state, "get_pp_group": lambda: group,
                    "is_pipeline_first_stage": lambda: stage == 0, "is_pipeline_last_stage": lambda: stage == stages - 1,
                    "get_pipeline_parallel_world_size": lambda: stages, "get_sequence_parallel_world_size": lambda: 1,
                    "get_sp_group": lambda: None,
                }
                for name in ("_sync_pipeline", "_init_async_pipeline", "_async_pipeline"):
                    setattr(Pipe, name, _lift_method_undecorated(path, name, cls, ns))
                pipe = Pipe()
                bar = _NS(update=lambda: None)
                latents = whole()
                timesteps = list(range(n_steps))
                extra = dict(text_ids=None, latent_image_ids=torch.zeros(patch_h * n_patch, 3), guidance=None) if flux else {}
                # the entry point's branch (pipeline_stable_diffusion_3.py:372-411, pipeline_flux.py:346-390)
                if n_patch > 1 and n_steps > warmup:
                    latents = pipe._sync_pipeline(latents=latents, prompt_embeds=prompt, pooled_prompt_embeds=None,
                                                  timesteps=timesteps[:warmup], num_warmup_steps=0, progress_bar=bar, **extra)
                    pipe._async_pipeline(latents=latents, prompt_embeds=prompt, pooled_prompt_embeds=None,
                                         timesteps=timesteps[warmup:], num_warmup_steps=0, progress_bar=bar, **extra)
                else:
                    pipe._sync_pipeline(latents=latents, prompt_embeds=prompt, pooled_prompt_embeds=None,
                                        timesteps=timesteps, num_warmup_steps=0, progress_bar=bar, sync_only=True, **extra)
                cases.append({"pipeline": family, "stages": stages, "stage": stage, "num_pipeline_patch": n_patch,
                              "steps": n_steps, "warmup": warmup, "events": events})
    with open(os.path.join(HERE, "pipefusion_order.json"), "w") as f:
        json.dump(cases, f, separators=(",", ":"))
    print("pipefusion_order.json written:", len(cases), "cases")


# ----------------------------------------------------------------------------- position-embedding rows per rank
def _runs(idx):
    """Maximal contiguous runs [start, end) of an increasing-by-one-within-run index list."""
    runs = []
    for v in idx:
        if runs and runs[-1][1] == v:
            runs[-1][1] = v + 1
        else:
            runs.append([v, v + 1])
    return runs


def gen_pos_embed_rows(ref):
    """Runs the reference's patch-embedding wrapper forward
    (model_executor/diffusion_executor/layers/embeddings.py:31-112) on a stand-in module whose projection is the
    identity on zeros and whose position table holds its own row numbers, with the patch metadata the reference's
    _calc_patches_metadata computes, and writes which table rows each rank adds: whole-image mode and every patch
    of patch mode."""
    log = logging.getLogger("golden")
    rs_path = os.path.join(ref, "hetu_dit/core/distributed/runtime_state.py")
    em_path = os.path.join(ref, "hetu_dit/model_executor/diffusion_executor/layers/embeddings.py")
    cases = []
    for (h, w, vae, patch, npp, sp) in [(1024, 1024, 8, 2, 4, 1), (1024, 1024, 8, 2, 4, 2), (1024, 1024, 8, 2, 4, 4),
                                        (512, 512, 8, 2, 2, 2), (1152, 896, 8, 2, 3, 2), (1024, 2048, 8, 2, 4, 2),
                                        (768, 768, 8, 2, 1, 1), (1024, 1024, 8, 2, 1, 8), (1536, 1536, 8, 2, 8, 1)]:
        for rank in range(sp):
            meta, _ = lift(rs_path, "_calc_patches_metadata", cls="DiTRuntimeState", namespace={
                "get_sequence_parallel_world_size": lambda sp=sp: sp,
                "get_sequence_parallel_rank": lambda rank=rank: rank, "logger": log})
            state = _NS(backbone_patch_size=patch, vae_scale_factor=vae,
                        input_config=_NS(height=h, width=w),
                        parallel_config=_NS(pp_config=_NS(num_pipeline_patch=npp)), patch_mode=False,
                        pipeline_patch_idx=0)
            meta(state)
            gh, gw = h // vae // patch, w // vae // patch
            table = torch.arange(gh * gw, dtype=torch.float32).reshape(1, gh * gw, 1)
            module = _NS(patch_size=patch, pos_embed_max_size=None, proj=lambda x: x, flatten=False, layer_norm=False,
                         pos_embed=table, height=gh, width=gw)
            fwd, _ = lift(em_path, "forward", cls="hetuDiTPatchEmbedWrapper",
                          namespace={"get_runtime_state": lambda: state, "torch": torch})
            wrapper = _NS(module=module)
            rec = {"height": h, "width": w, "vae": vae, "patch": patch, "num_pipeline_patch": state.num_pipeline_patch,
                   "sp_world": sp, "sp_rank": rank,
                   "bounds": [list(b) for b in state.pp_patches_token_start_end_idx_global]}
            n_local = sum(e - s for s, e in state.pp_patches_token_start_end_idx_global)
            # the wrapper reads the latent width in pixels from the last dimension
            rows = fwd(wrapper, torch.zeros(1, n_local, w // vae))[0, :, 0].long().tolist()
            rec["whole_image_rows"] = _runs(rows)
            state.patch_mode = True
            rec["patch_rows"] = []
            for p in range(state.num_pipeline_patch):
                state.pipeline_patch_idx = p
                s, e = state.pp_patches_token_start_end_idx_global[p]
                rec["patch_rows"].append(_runs(fwd(wrapper, torch.zeros(1, e - s, w // vae))[0, :, 0].long().tolist()))
            cases.append(rec)
    with open(os.path.join(HERE, "pos_embed_rows.json"), "w") as f:
        json.dump(cases, f, separators=(",", ":"))
    print("pos_embed_rows.json written:", len(cases), "cases")


# ----------------------------------------------------------------------------- attention processors
def _find_class_anywhere(tree, cls):
    for node in ast.walk(tree):
        if isinstance(node, ast.ClassDef) and node.name == cls:
            return node
    raise KeyError(cls)


def gen_attn_processors(ref):
    """Runs the __call__ of the reference's attention processors
    (model_executor/diffusion_executor/layers/attention_processor.py: hetuDiTJointAttnProcessor2_0 :657,
    hetuDiTFluxAttnProcessor2_0 :824, hetuDiTCogVideoXAttnProcessor2_0 :1022, hetuDiTHunyuanVideoAttnProcessor2_0
    :1373) on CPU in fp32 -- their scaled_dot_product_attention branch, one GPU, no pipeline patches -- with a
    stand-in for the diffusers Attention module that holds seeded projections and QK norms, and writes inputs,
    weights and outputs. The stand-in restates only diffusers' RMSNorm (x * rsqrt(mean(x^2) + eps) * weight)."""
    from typing import Optional, Tuple, Union
    import torch.nn as nn
    import torch.nn.functional as F
    path = os.path.join(ref, "hetu_dit/model_executor/diffusion_executor/layers/attention_processor.py")
    with open(path) as f:
        tree = ast.parse(f.read())
    rope_fn, _ = lift(path, "apply_rotary_emb", namespace={"torch": torch, "Union": Union, "Tuple": Tuple})

    class RMSNorm(nn.Module):
        def __init__(self, dim, eps):
            super().__init__()
            self.weight, self.eps = nn.Parameter(torch.ones(dim)), eps

        def forward(self, x):
            return x * torch.rsqrt(x.float().pow(2).mean(-1, keepdim=True) + self.eps) * self.weight

    state = _NS(max_condition_sequence_length=0, split_text_embed_in_sp=False, num_pipeline_patch=1)
    cache = _NS(update_and_get_kv_cache=lambda new_kv, layer, slice_dim, layer_type: new_kv)
    ns = {"torch": torch, "F": F, "Optional": Optional, "Attention": object, "HAS_LONG_CTX_ATTN": False,
          "HAS_FLASH_ATTN": False, "get_sequence_parallel_world_size": lambda: 1,
          "get_tensor_model_parallel_world_size": lambda: 1, "get_pipeline_parallel_world_size": lambda: 1,
          "get_runtime_state": lambda: state, "get_cache_manager": lambda: cache, "apply_rotary_emb": rope_fn}

    def call_of(cls):
        node = next(n for n in _find_class_anywhere(tree, cls).body
                    if isinstance(n, ast.FunctionDef) and n.name == "__call__")
        scope = dict(ns)
        exec(compile(ast.Module(body=[node], type_ignores=[]), path, "exec"), scope)
        return scope["__call__"]

    H, D, B, S_img, S_txt = 2, 16, 2, 10, 6
    d = H * D
    gen = torch.Generator().manual_seed(77)

    def attn_module(norm, joint):
        a = _NS(heads=H, is_cross_attention=False, spatial_norm=None, group_norm=None, norm_cross=False)
        names = ["to_q", "to_k", "to_v"] + (["add_q_proj", "add_k_proj", "add_v_proj"] if joint else [])
        for n in names:
            lin = nn.Linear(d, d)
            lin.weight.data = torch.randn(d, d, generator=gen) / d ** 0.5
            lin.bias.data = torch.randn(d, generator=gen) * 0.1
            setattr(a, n, lin)
        if not joint:
            a.add_q_proj = a.add_k_proj = a.add_v_proj = None
        for n in ["norm_q", "norm_k"] + (["norm_added_q", "norm_added_k"] if joint else []):
            if norm == "rms":
                m = RMSNorm(D, 1e-6)
                m.weight.data = torch.rand(D, generator=gen) + 0.5
            elif norm == "layer":
                m = nn.LayerNorm(D, eps=1e-6)
                m.weight.data = torch.rand(D, generator=gen) + 0.5
                m.bias.data = torch.randn(D, generator=gen) * 0.1
            else:
                m = None
            setattr(a, n, m)
        if not joint:
            a.norm_added_q = a.norm_added_k = None
        return a

    def rope(rows):
        ang = torch.rand(rows, D // 2, generator=gen) * 6.28
        return torch.cos(ang).repeat_interleave(2, dim=-1), torch.sin(ang).repeat_interleave(2, dim=-1)

    data = {"spec": np.array(json.dumps({"heads": H, "head_dim": D, "batch": B, "s_img": S_img, "s_txt": S_txt}))}

    def record(case, a, inputs, outputs, rope_tab=None):
        for n in ("to_q", "to_k", "to_v", "add_q_proj", "add_k_proj", "add_v_proj"):
            m = getattr(a, n, None)
            if m is not None:
                data[f"{case}/{n}.weight"], data[f"{case}/{n}.bias"] = m.weight.detach().numpy(), m.bias.detach().numpy()
        for n in ("norm_q", "norm_k", "norm_added_q", "norm_added_k"):
            m = getattr(a, n, None)
            if m is not None:
                data[f"{case}/{n}.weight"] = m.weight.detach().numpy()
                if getattr(m, "bias", None) is not None:
                    data[f"{case}/{n}.bias"] = m.bias.detach().numpy()
        for k, v in inputs.items():
            data[f"{case}/in.{k}"] = v.numpy()
        for k, v in outputs.items():
            data[f"{case}/out.{k}"] = v.detach().numpy()
        if rope_tab is not None:
            data[f"{case}/cos"], data[f"{case}/sin"] = rope_tab[0].numpy(), rope_tab[1].numpy()

    with torch.no_grad():
        hid = torch.randn(B, S_img, d, generator=gen)
        txt = torch.randn(B, S_txt, d, generator=gen)
        # SD3: [image; text], no QK norm, no rotary embedding
        a = attn_module(None, True)
        img_o, txt_o = call_of("hetuDiTJointAttnProcessor2_0")(_NS(), a, hid, txt)
        record("joint_sd3", a, {"hidden": hid, "encoder": txt}, {"image": img_o, "text": txt_o})
        # Flux double block: [text; image], RMSNorm, rotary rows for text and image
        a = attn_module("rms", True)
        tab = rope(S_txt + S_img)
        img_o, txt_o = call_of("hetuDiTFluxAttnProcessor2_0")(_NS(), a, hid, txt, None, tab)
        record("flux_double", a, {"hidden": hid, "encoder": txt}, {"image": img_o, "text": txt_o}, tab)
        # Flux single block: joint rows [text; image] come in as hidden_states
        a = attn_module("rms", False)
        state.max_condition_sequence_length = S_txt
        joint = torch.cat([txt, hid], dim=1)
        out = call_of("hetuDiTFluxAttnProcessor2_0")(_NS(), a, joint, None, None, tab)
        record("flux_single", a, {"hidden": joint}, {"joint": out}, tab)
        # CogVideoX: [text; video], LayerNorm QK norm, rotary rows for the video only
        a = attn_module("layer", False)
        tab_v = rope(S_img)
        out = call_of("hetuDiTCogVideoXAttnProcessor2_0")(_NS(), a, hid, txt, None, tab_v)
        record("cogvideox", a, {"hidden": hid, "encoder": txt}, {"joint": out}, tab_v)
        # HunyuanVideo double block: [video; text], RMSNorm, rotary rows for the video only
        a = attn_module("rms", True)
        out = call_of("hetuDiTHunyuanVideoAttnProcessor2_0")(_NS(), a, hid, txt, None, tab_v)
        record("hunyuan_double", a, {"hidden": hid, "encoder": txt}, {"joint": out}, tab_v)
        # HunyuanVideo single block: [video; text] concatenated by the processor
        a = attn_module("rms", False)
        out = call_of("hetuDiTHunyuanVideoAttnProcessor2_0")(_NS(), a, hid, txt, None, tab_v)
        record("hunyuan_single", a, {"hidden": hid, "encoder": txt}, {"joint": out}, tab_v)
    np.savez_compressed(os.path.join(HERE, "attn_processors.npz"), **data)
    print("attn_processors.npz written:", len(data), "arrays")


# ----------------------------------------------------------------------------- pipeline stage split
def gen_stage_split(ref):
    """Runs the reference's _split_transformer_blocks
    (model_executor/diffusion_executor/models/transformers/base_transformer.py:65-146) on a stand-in transformer with
    numbered double and single blocks and writes, per (block counts, stages, stage, explicit per-stage counts), which
    blocks the stage keeps and its after_flags."""
    from typing import List
    import torch.nn as nn
    path = os.path.join(ref, "hetu_dit/model_executor/diffusion_executor/models/transformers/base_transformer.py")

    class Block(nn.Module):
        def __init__(self, i):
            super().__init__()
            self.i = i

    cases = []
    for (n_double, n_single, stages, counts) in [
            (24, 0, 1, None), (24, 0, 2, None), (24, 0, 4, None), (24, 0, 5, None), (24, 0, 4, [3, 9, 6, 6]),
            (19, 38, 2, None), (19, 38, 4, None), (19, 38, 8, None), (19, 38, 3, None), (19, 38, 4, [19, 10, 14, 14]),
            (19, 38, 4, [5, 14, 19, 19]), (2, 3, 2, None), (2, 3, 5, None), (20, 40, 8, None), (42, 0, 8, None)]:
        for stage in range(stages):
            state = _NS(parallel_config=_NS(pp_config=_NS(attn_layer_num_for_pp=counts)))
            ns = {"nn": nn, "List": List, "get_runtime_state": lambda state=state: state,
                  "get_pipeline_parallel_rank": lambda stage=stage: stage,
                  "get_pipeline_parallel_world_size": lambda stages=stages: stages,
                  "StageInfo": lambda: _NS(after_flags={})}
            fn, _ = lift(path, "_split_transformer_blocks", cls="hetuDiTDiffusionTransformerBaseWrapper", namespace=ns)
            t = nn.Module()
            t.transformer_blocks = nn.ModuleList([Block(i) for i in range(n_double)])
            names = ["transformer_blocks"]
            if n_single:
                t.single_transformer_blocks = nn.ModuleList([Block(i) for i in range(n_single)])
                names.append("single_transformer_blocks")
            self = _NS()
            fn(self, t, names)
            cases.append({"n_double": n_double, "n_single": n_single, "stages": stages, "stage": stage,
                          "attn_layer_num_for_pp": counts,
                          "double": [b.i for b in t.transformer_blocks],
                          "single": [b.i for b in t.single_transformer_blocks] if n_single else [],
                          "after_flags": dict(self.stage_info.after_flags)})
    with open(os.path.join(HERE, "stage_split.json"), "w") as f:
        json.dump(cases, f, separators=(",", ":"))
    print("stage_split.json written:", len(cases), "cases")


# ----------------------------------------------------------------------------- scheduler step
def gen_scheduler_step(ref):
    """Runs the step() of the reference's flow-matching Euler scheduler wrapper
    (model_executor/diffusion_executor/schedulers/scheduling_flow_match_euler_discrete.py:22-129) over the patches
    of a few steps: the new sample per call and when the step index advances (after the last patch only, in patch
    mode). Inputs are 16-bit as the pipelines pass them; the wrapper computes in fp32 and rounds once."""
    from typing import Optional, Tuple, Union
    path = os.path.join(ref, "hetu_dit/model_executor/diffusion_executor/schedulers/"
                             "scheduling_flow_match_euler_discrete.py")
    with open(path) as f:
        tree = ast.parse(f.read())
    node = next(n for n in _find_class_anywhere(tree, "hetuDiTFlowMatchEulerDiscreteSchedulerWrapper").body
                if isinstance(n, ast.FunctionDef) and n.name == "step")
    node.decorator_list = []
    state = _NS(patch_mode=True, pipeline_patch_idx=0, num_pipeline_patch=4)
    ns = {"torch": torch, "Optional": Optional, "Tuple": Tuple, "Union": Union,
          "FlowMatchEulerDiscreteSchedulerOutput": lambda prev_sample: prev_sample,
          "get_runtime_state": lambda: state,
          "randn_tensor": lambda shape, dtype, device, generator: torch.zeros(shape, dtype=dtype, device=device)}
    exec(compile(ast.Module(body=[node], type_ignores=[]), path, "exec"), ns)
    step = ns["step"]
    gen = torch.Generator().manual_seed(5)
    n_steps = 6
    s = torch.linspace(1.0, 1.0 / n_steps, n_steps, dtype=torch.float64)
    sigmas = torch.cat([3.0 * s / (1 + 2.0 * s), torch.zeros(1, dtype=torch.float64)]).float()
    data = {"sigmas": sigmas.numpy()}
    calls = []
    for dtype, tag in ((torch.bfloat16, "bf16"), (torch.float16, "fp16")):
        sched = _NS(sigmas=sigmas, step_index=0, _step_index=0)
        for mode, patches in ((False, 1), (True, 4)):
            state.patch_mode, state.num_pipeline_patch = mode, patches
            for it in range(2):
                for p in range(patches):
                    state.pipeline_patch_idx = p
                    sched.step_index = sched._step_index
                    mo = torch.randn(2, 24, 16, generator=gen).to(dtype)
                    x = torch.randn(2, 24, 16, generator=gen).to(dtype)
                    before = sched._step_index
                    out = step(sched, mo, 0.5, x, return_dict=False)[0]
                    k = f"{tag}/{len(calls)}"
                    data[k + "/model_output"], data[k + "/sample"] = mo.float().numpy(), x.float().numpy()
                    data[k + "/prev_sample"] = out.float().numpy()
                    calls.append({"key": k, "dtype": tag, "step_index": before, "patch_mode": mode, "patch": p,
                                  "patches": patches, "advanced": sched._step_index - before})
    data["calls"] = np.array(json.dumps(calls))
    np.savez_compressed(os.path.join(HERE, "scheduler_step.npz"), **data)
    print("scheduler_step.npz written:", len(calls), "calls")


# ----------------------------------------------------------------------------- stage forward of the transformer wrappers
STAND_IN_HIDDEN = 8


def stand_in_double(i, hidden, text, temb):
    """Arithmetic of stand-in joint block i (repeated in tests/test_host_logic.py): both streams mix, so that a
    wrong text source, block order or stage boundary changes the result."""
    h = hidden * 1.5 + text.mean(1, keepdim=True) + temb[:, None] + (i + 1)
    c = text * 0.5 + hidden.mean(1, keepdim=True) * 0.25 - (i + 1)
    return h, c


def stand_in_single(j, x, temb):
    """Stand-in single block j on the joined rows: row-dependent, so that the join order matters."""
    rows = torch.arange(x.shape[1], dtype=x.dtype)[None, :, None]
    return x * 1.25 + rows * 0.01 * (j + 1) + temb[:, None]


def stand_in_out_norm(hidden, temb):
    x = torch.nn.functional.silu(temb)[:, None]
    return torch.nn.functional.layer_norm(hidden, (hidden.shape[-1],), eps=1e-6) * (1 + 0.1 * x) + 0.2 * x


def gen_stage_forward(ref):
    """Runs forward() of the reference's SD3 and Flux transformer wrappers
    (model_executor/diffusion_executor/models/transformers/transformer_sd3.py:43-198, transformer_flux.py:45-217) for
    every stage of 1- to 4-stage pipelines, on stand-in embedders / blocks / output layers with the arithmetic above,
    the block lists cut by the reference's own _split_transformer_blocks. Whole-image calls and patch-mode calls
    (patches 0, 1, 2 in order: the SD3 wrapper keeps each block's text input of patch 0 and re-uses it for the later
    patches). Written per call: the stage's inputs and outputs."""
    from typing import Any, Dict, List, Optional, Union
    import torch.nn as nn
    base = os.path.join(ref, "hetu_dit/model_executor/diffusion_executor/models/transformers")
    d = STAND_IN_HIDDEN

    class Double(nn.Module):
        def __init__(self, i):
            super().__init__()
            self.i = i

        def forward(self, hidden_states, encoder_hidden_states, temb, image_rotary_emb=None):
            h, c = stand_in_double(self.i, hidden_states, encoder_hidden_states, temb)
            return c, h

    class Single(nn.Module):
        def __init__(self, j):
            super().__init__()
            self.j = j

        def forward(self, hidden_states, temb, image_rotary_emb=None):
            return stand_in_single(self.j, hidden_states, temb)

    def temb_of(*a):                       # (timestep, pooled) or (timestep, guidance, pooled)
        pooled = a[-1]
        return 0.125 + 0.0625 * (len(a) == 3) + pooled.sum(-1, keepdim=True).expand(-1, d)

    gen = torch.Generator().manual_seed(11)
    data, calls = {}, []
    for model, n_double, n_single, cls, fname in (("sd3", 5, 0, "hetuDiTSD3Transformer2DWrapper", "transformer_sd3.py"),
                                                   ("flux", 3, 4, "hetuDiTFluxTransformer2DWrapper",
                                                    "transformer_flux.py")):
        for stages in (1, 2, 3, 4):
            state = _NS(parallel_config=_NS(pp_config=_NS(attn_layer_num_for_pp=None)), patch_mode=False,
                        pipeline_patch_idx=0)
            wrappers = []
            for stage in range(stages):
                ns = {"nn": nn, "List": List, "get_runtime_state": lambda: state,
                      "get_pipeline_parallel_rank": lambda stage=stage: stage,
                      "get_pipeline_parallel_world_size": lambda stages=stages: stages,
                      "StageInfo": lambda: _NS(after_flags={})}
                split, _ = lift(os.path.join(base, "base_transformer.py"), "_split_transformer_blocks",
                                cls="hetuDiTDiffusionTransformerBaseWrapper", namespace=ns)
                t = nn.Module()
                t.transformer_blocks = nn.ModuleList([Double(i) for i in range(n_double)])
                names = ["transformer_blocks"]
                if n_single:
                    t.single_transformer_blocks = nn.ModuleList([Single(j) for j in range(n_single)])
                    names.append("single_transformer_blocks")
                w = _NS(training=False, gradient_checkpointing=False, config=_NS(patch_size=1), out_channels=d)
                split(w, t, names)
                w.transformer_blocks = t.transformer_blocks
                w.single_transformer_blocks = t.single_transformer_blocks if n_single else []
                w.encoder_hidden_states_cache = [None] * len(w.transformer_blocks)
                w.pos_embed = (lambda h: h * 2.0 + 1.0) if model == "sd3" else (lambda ids: None)
                w.x_embedder = lambda h: h * 2.0 + 1.0
                w.context_embedder = lambda c: c * 3.0 - 1.0
                w.time_text_embed = temb_of
                w.norm_out = stand_in_out_norm
                w.proj_out = lambda h: h * 7.0
                w._get_patch_height_width = lambda: (1, 6)
                fns = {"torch": torch, "Optional": Optional, "Dict": Dict, "Any": Any, "Union": Union,
                       "Transformer2DModelOutput": lambda sample: sample, "USE_PEFT_BACKEND": False,
                       "logger": logging.getLogger("ref"), "get_runtime_state": lambda: state,
                       "is_pipeline_first_stage": lambda stage=stage: stage == 0,
                       "is_pipeline_last_stage": lambda stage=stage, stages=stages: stage == stages - 1,
                       "is_torch_version": lambda *a: True}
                fwd = _lift_method_undecorated(os.path.join(base, fname), "forward", cls, fns)
                wrappers.append((w, fwd))
            pooled = torch.randn(2, 4, generator=gen, dtype=torch.float64) * 0.1
            text0 = torch.randn(2, 3, d, generator=gen, dtype=torch.float64)
            for mode, patches in (("whole", [None]), ("patch", [0, 1, 2])):
                for patch in patches:
                    state.patch_mode = mode == "patch"
                    state.pipeline_patch_idx = patch or 0
                    h = torch.randn(2, 6, d, generator=gen, dtype=torch.float64)
                    c = text0 if not patch else text0 + 100.0       # later patches: the blocks must not read this
                    for stage, (w, fwd) in enumerate(wrappers):
                        kw = dict(hidden_states=h, encoder_hidden_states=c, pooled_projections=pooled,
                                  timestep=torch.full((2,), 0.5, dtype=torch.float64), return_dict=False)
                        if model == "flux":
                            kw.update(img_ids=torch.zeros(6, 3), txt_ids=torch.zeros(3, 3),
                                      guidance=torch.full((2,), 3.5, dtype=torch.float64))
                        record = {}
                        if stage == stages - 1:
                            w.proj_out = lambda x, record=record: record.setdefault("tokens", x * 7.0)
                        out_h, out_c = fwd(w, **kw)[0]
                        if stage == stages - 1:
                            out_h = record["tokens"]            # the token form, before the SD3 wrapper's unpatchify
                        k = f"{model}/pp{stages}/{mode}{'' if patch is None else patch}/s{stage}"
                        data[k + "/in_h"], data[k + "/in_c"] = h.numpy(), c.numpy()
                        data[k + "/out_h"] = out_h.numpy()
                        if out_c is not None:
                            data[k + "/out_c"] = out_c.numpy()
                        calls.append({"key": k, "model": model, "stages": stages, "stage": stage, "mode": mode,
                                      "patch": patch, "n_double": n_double, "n_single": n_single,
                                      "text_out": out_c is not None})
                        h, c = out_h, (out_c if out_c is not None else c)
            data[f"{model}/pp{stages}/pooled"] = pooled.numpy()
    data["calls"] = np.array(json.dumps(calls))
    np.savez_compressed(os.path.join(HERE, "stage_forward.npz"), **data)
    print("stage_forward.npz written:", len(calls), "calls")


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="root of a Hetu-DiT checkout")
    ap.add_argument("--only", default="")
    a = ap.parse_args()
    logging.basicConfig(level=logging.ERROR)
    torch.set_num_threads(2)
    if a.only in ("", "bookkeeping"):
        gen_bookkeeping(a.reference)
    if a.only in ("", "rope"):
        gen_rope(a.reference)
    if a.only in ("", "usp"):
        gen_usp(a.reference)
    if a.only.startswith("usp:"):                       # e.g. --only usp:ulysses_
        gen_usp(a.reference, a.only[4:])
    if a.only in ("", "scheduler_step"):
        gen_scheduler_step(a.reference)
    if a.only in ("", "stage_forward"):
        gen_stage_forward(a.reference)
    if a.only in ("", "stage_split"):
        gen_stage_split(a.reference)
    if a.only in ("", "attn_processors"):
        gen_attn_processors(a.reference)
    if a.only in ("", "pos_embed_rows"):
        gen_pos_embed_rows(a.reference)
    if a.only in ("", "pipefusion_order"):
        gen_pipefusion_order(a.reference)
