"""CPU oracle: integer bookkeeping of the Hetu-DiT denoising hot path.

TEST INFRASTRUCTURE ONLY. Nothing under hetu_dit_b200/ may import this module;
it is the checker that tests/, __graft_entry__.smoke() and bench.py's CPU
baseline compare the product against.

Every function restates one reference function in plain Python (paths are
relative to the reference repository root). Parity is pinned: the fixtures in
tests/golden/bookkeeping.json were produced by running the reference's own
functions (lifted from its source files, see tests/golden/make_golden.py) and
tests/test_oracle_golden.py checks this restatement against them bit for bit.
"""
from itertools import combinations


# ---------------------------------------------------------------------------
# PipeFusion patch metadata
# hetu_dit/core/distributed/runtime_state.py:333-446 (_calc_patches_metadata)
# hetu_dit/core/distributed/runtime_state.py:448-555 (_calc_cogvideox_patches_metadata)
# ---------------------------------------------------------------------------
def calc_patches_metadata(height, width, vae_scale_factor, patch_size, num_pipeline_patch, sp_world, sp_rank,
                          check_last_patch=True):
    """Patch bookkeeping for one SP rank.

    The latent height is cut into `num_pipeline_patch` bands whose height is
    rounded up to a multiple of patch_size * sp_world (which may lower the band
    count); every SP rank owns one 1/sp_world slice of every band. The image
    variant raises when the last band is not such a multiple
    (runtime_state.py:378-384); the CogVideoX variant (check_last_patch=False)
    does not.
    """
    lat_h = height // vae_scale_factor
    lat_w = width // vae_scale_factor
    if lat_h % sp_world != 0:
        raise ValueError("The height of the input is not divisible by the number of sequence parallel devices")
    unit = patch_size * sp_world
    band = -(-lat_h // num_pipeline_patch)
    band = -(-band // unit) * unit
    n_band = -(-lat_h // band)
    bands = [band] * (n_band - 1)
    last = lat_h - band * (n_band - 1)
    if check_last_patch and last % unit != 0:
        raise ValueError("last pipeline patch height is not a multiple of patch_size * num_sp_patches")
    bands.append(last)

    # The reference flattens rank-major (rank outer, band inner) but then reads the
    # flat list back as if it were band-major; both steps are reproduced as they are.
    flat_h = [b // sp_world for _ in range(sp_world) for b in bands]
    flat_start = [0]
    for h in flat_h:
        flat_start.append(flat_start[-1] + h)
    per_band_h = [flat_h[p * sp_world:(p + 1) * sp_world] for p in range(n_band)]
    per_band_start = [flat_start[p * sp_world:(p + 1) * sp_world + 1] for p in range(n_band)]

    heights = [hs[sp_rank] for hs in per_band_h]
    start_local = [0]
    for h in heights:
        start_local.append(start_local[-1] + h)
    se_global = [st[sp_rank:sp_rank + 2] for st in per_band_start]
    tokens_per_row = lat_w // patch_size
    tok_se_global = [[tokens_per_row * (s // patch_size), tokens_per_row * (e // patch_size)] for s, e in se_global]
    tok_num = [e - s for s, e in tok_se_global]
    tok_start_local = [0]
    for n in tok_num:
        tok_start_local.append(tok_start_local[-1] + n)
    return {
        "num_pipeline_patch": n_band,
        "pp_patches_height": heights,
        "pp_patches_start_idx_local": start_local,
        "pp_patches_start_end_idx_global": se_global,
        "pp_patches_token_start_idx_local": tok_start_local,
        "pp_patches_token_start_end_idx_global": tok_se_global,
        "pp_patches_token_num": tok_num,
    }


def calc_cogvideox_patches_metadata(height, width, vae_scale_factor_spatial, patch_size, num_pipeline_patch, sp_world,
                                    sp_rank):
    """runtime_state.py:448-555 -- same arithmetic, no check on the last band."""
    return calc_patches_metadata(height, width, vae_scale_factor_spatial, patch_size, num_pipeline_patch, sp_world,
                                 sp_rank, check_last_patch=False)


def next_patch(patch_mode, idx, num_pipeline_patch):
    """runtime_state.py:258-264."""
    if not patch_mode:
        return 0
    idx += 1
    return 0 if idx == num_pipeline_patch else idx


# ---------------------------------------------------------------------------
# Rank groups
# hetu_dit/core/distributed/utils.py:4-110 (generate_masked_orthogonal_rank_groups)
# hetu_dit/core/distributed/utils.py:113-188 (RankGenerator)
# ---------------------------------------------------------------------------
def orthogonal_rank_groups(world_size, sizes, mask):
    """Groups of ranks that vary exactly the masked axes of a mixed-radix rank index."""
    strides = [1]
    for s in sizes:
        strides.append(strides[-1] * s)
    in_axes = [(s, strides[i]) for i, s in enumerate(sizes) if mask[i]]
    out_axes = [(s, strides[i]) for i, s in enumerate(sizes) if not mask[i]]

    def expand(index, axes):
        total, div = 0, 1
        for size, stride in axes:
            total += ((index // div) % size) * stride
            div *= size
        return total

    group_size = 1
    for s, _ in in_axes:
        group_size *= s
    return [[expand(r, in_axes) + expand(g, out_axes) for r in range(group_size)]
            for g in range(world_size // group_size)]


def rank_generator_groups(tp, sp, pp, cfg, dp, token, order="tp-sp-pp-cfg-dp", rank_offset=0):
    names = {"tp": tp, "sp": sp, "pp": pp, "cfg": cfg, "dp": dp}
    order_tokens = order.lower().split("-")
    for name, size in names.items():
        if name not in order_tokens:
            if size != 1:
                raise RuntimeError(f"size of {name} is {size} but it is missing from the order")
            order_tokens.append(name)
    sizes = [names[t] for t in order_tokens]
    wanted = token.split("-")
    mask = [t in wanted for t in order_tokens]
    groups = orthogonal_rank_groups(tp * sp * pp * cfg * dp, sizes, mask)
    return [[r + rank_offset for r in g] for g in groups]


def seq_parallel_rank_groups(ulysses, ring, world_size, ranks, use_ulysses_low=True):
    """hetu_dit/core/distributed/parallel_state.py:642-749 (set_seq_parallel_pg), rank lists only.

    Returns (ulysses_groups, ring_groups) in creation order. `ranks` are the
    global ranks the plan is placed on; position i of sorted(ranks) plays local rank i.
    """
    sp = ulysses * ring
    assert world_size % sp == 0
    rank_map = sorted(ranks)
    u_groups, r_groups = [], []
    for d in range(world_size // sp):
        off = d * sp
        if use_ulysses_low:
            for i in range(ring):
                u_groups.append([rank_map[r] for r in range(i * ulysses + off, (i + 1) * ulysses + off)])
            for i in range(ulysses):
                r_groups.append([rank_map[r] for r in range(i + off, sp + off, ulysses)])
        else:
            for i in range(ulysses):
                r_groups.append([rank_map[r] for r in range(i * ring + off, (i + 1) * ring + off)])
            for i in range(ring):
                u_groups.append([rank_map[r] for r in range(i + off, sp + off, ring)])
    return u_groups, r_groups


def rank_combinations(world_size, valid_degrees=(1, 2, 4, 8), base_num=0):
    """parallel_state.py:833-847 (_generate_rank_combinations)."""
    out = []
    for degree in valid_degrees:
        if degree > world_size:
            continue
        out.extend([[r + base_num for r in c] for c in combinations(range(world_size), degree)])
    return out


def group_partitions(ranks):
    """parallel_state.py:849-908 (_generate_group_ranks): every split of `ranks` into equal power-of-two groups."""
    def split(rs, size):
        if len(rs) == size:
            return [[list(rs)]]
        first, rest = rs[0], rs[1:]
        res = []
        for others in combinations(rest, size - 1):
            head = [first] + list(others)
            remaining = [r for r in rs if r not in head]
            for tail in split(remaining, size):
                res.append([head] + tail)
        return res

    n = len(ranks)
    if n == 1:
        return [[list(ranks)]]
    out = []
    for i in range(n.bit_length()):
        part = 1 << i
        if part > n:
            break
        if n % part == 0:
            out.extend(split(list(ranks), part))
    return out


# ---------------------------------------------------------------------------
# Parameter-slice ranges
# ---------------------------------------------------------------------------
def gpu_metadata(pp_rank, pp_world, tp_rank, tp_world):
    """hetu_dit/utils.py:788-828 (get_gpu_metadata): fractional TP / PP ranges of one rank."""
    t = 1.0 / tp_world
    ts = tp_rank * t
    p = 1.0 / pp_world
    ps = pp_rank * p
    return {"tensor_parallel": (ts, ts + t), "pipeline_parallel": (ps, ps + p)}


def range_to_indices_round(rng, total):
    """hetu_dit/utils.py:437-441: round() based, used by the `base` strategy."""
    return round(rng[0] * total), round(rng[1] * total)


def range_to_indices_trunc(rng, total):
    """hetu_dit/model_executor/cache/base_cache.py:213-235: int() truncation, clamp, end snap at 1.0."""
    if total == 0:
        return 0, 0
    s = max(0, min(int(rng[0] * total), total))
    e = max(0, min(int(rng[1] * total), total))
    if s > e:
        e = s
    elif rng[1] == 1.0 and e < total:
        e = total
    return s, e


ROW_SPLIT_KEYS = ("to_q", "to_k", "to_v", "add_k_proj", "add_q_proj", "add_v_proj")
COLUMN_SPLIT_KEYS = ("to_out", "to_add_out")
ADJUSTED_LINEARS = frozenset(
    f"{a}.module.{n}" for a in ("attn", "attn1")
    for n in ("to_q", "to_k", "to_v", "add_k_proj", "add_q_proj", "add_v_proj", "to_add_out", "to_out.0")
) | frozenset(("ff.module.net.0.proj", "ff.module.net.2", "ff_context.module.net.0.proj", "ff_context.module.net.2"))


def tp_split_type(name):
    """hetu_dit/model_executor/cache/transformer_cache.py:113-154: 'row' / 'column' / None."""
    if name not in ADJUSTED_LINEARS:
        return None
    low = name.lower()
    if any(k in low for k in ROW_SPLIT_KEYS):
        return "row"
    if any(k in low for k in COLUMN_SPLIT_KEYS):
        return "column"
    if "net.0.proj" in low:
        return "row"
    if "net.2" in low:
        return "column"
    return "row"


def needed_pieces(block_indices, linears, cached_tp, target_tp, slice_bias=True):
    """Plan construction of base_cache.py:331-455.

    block_indices: blocks the new plan needs, in order.
    linears: {block_index: [(name, out_features, in_features, has_bias), ...]} in named_modules order.
    cached_tp: {block_index: (start, end)} fractional TP range of blocks already on this GPU.
    Returns a list of dicts with the NeededPiece fields (base_cache.py:20-38).
    """
    pieces = []
    uid = 0
    for idx in block_indices:
        cached = cached_tp.get(idx)
        for name, out_f, in_f, has_bias in linears[idx]:
            kind = tp_split_type(name)
            if kind is None:
                continue
            full, dim = (out_f, 0) if kind == "row" else (in_f, 1)
            ns, ne = range_to_indices_trunc(target_tp, full)
            if ne <= ns:
                continue
            if cached is not None:
                os_, oe = range_to_indices_trunc(cached, full)
                ov_s, ov_e = max(ns, os_), min(ne, oe)
            else:
                ov_s, ov_e = ns, ns
            gaps = []
            if ov_s > ns:
                gaps.append((ns, ov_s))
            if ov_e < ne:
                gaps.append((ov_e, ne))
            for gs, ge in gaps:
                if ge <= gs:
                    continue
                uid += 1
                pieces.append(dict(uid=uid, block_index=idx, layer_path=name, tensor_type="weight", split_dim=dim,
                                   full_size=full, abs_start_idx=gs, abs_end_idx=ge, dest_offset=gs - ns))
                if slice_bias and kind == "row" and has_bias:
                    bs, _ = range_to_indices_trunc(target_tp, out_f)
                    b0 = bs + (gs - ns)
                    b1 = b0 + (ge - gs)
                    if b1 > b0:
                        uid += 1
                        pieces.append(dict(uid=uid, block_index=idx, layer_path=name, tensor_type="bias", split_dim=dim,
                                           full_size=out_f, abs_start_idx=b0, abs_end_idx=b1, dest_offset=b0 - bs))
    return pieces


def can_provide(piece, holder_tp):
    """worker/worker.py:2126-2132: a peer serves a piece only if its slice covers the whole span."""
    s, e = range_to_indices_trunc(holder_tp, piece["full_size"])
    return s <= piece["abs_start_idx"] and e >= piece["abs_end_idx"]


def piece_copy_descriptor(piece, holder_tp, src_shape, dst_shape, elem_size):
    """Byte-level 2-D copy a piece stands for.

    Source side: worker/worker.py:2354-2403; destination side:
    core/distributed/nixl_manager.py:209-252. Returns
    (src_offset_bytes, dst_offset_bytes, rows, row_bytes, src_pitch, dst_pitch)
    for contiguous (rows, cols) source and destination tensors.
    """
    my_s, _ = range_to_indices_trunc(holder_tp, piece["full_size"])
    rel = piece["abs_start_idx"] - my_s
    span = piece["abs_end_idx"] - piece["abs_start_idx"]
    if piece["tensor_type"] == "bias":
        return rel * elem_size, piece["dest_offset"] * elem_size, 1, span * elem_size, 0, 0
    src_pitch = src_shape[1] * elem_size
    dst_pitch = dst_shape[1] * elem_size
    if piece["split_dim"] == 0:
        return rel * src_pitch, piece["dest_offset"] * dst_pitch, 1, span * src_pitch, 0, 0
    return rel * elem_size, piece["dest_offset"] * elem_size, src_shape[0], span * elem_size, src_pitch, dst_pitch


# ---------------------------------------------------------------------------
# Stale-KV cache indices
# hetu_dit/core/resource_manager/cache_manager.py:117-206
# ---------------------------------------------------------------------------
def kv_cache_write_range(patch_mode, num_pipeline_patch, patch_idx, tok_start_local, ulysses_world=1,
                         sequence_parallel=False):
    """Token range of the stale-KV buffer a patch overwrites, or None for a whole-buffer store.

    naive cache (cache_manager.py:117-149): [tok_start[p], tok_start[p+1]);
    sequence-parallel cache (:186-205): the same range scaled by the Ulysses degree.
    """
    if num_pipeline_patch == 1 or not patch_mode:
        return None
    scale = ulysses_world if sequence_parallel else 1
    return scale * tok_start_local[patch_idx], scale * tok_start_local[patch_idx + 1]


def sp_warmup_kv_order(ulysses_world, tok_num):
    """cache_manager.py:172-183: source index ranges, in the order the warm-up cache concatenates them.

    The gathered K/V holds one chunk per Ulysses rank; each chunk is split by
    patch token counts and the pieces are laid out rank-major, patch-minor --
    i.e. in unchanged order. Returns [(start, end), ...] into the gathered sequence.
    """
    per_rank = sum(tok_num)
    out = []
    for r in range(ulysses_world):
        off = r * per_rank
        for n in tok_num:
            out.append((off, off + n))
            off += n
    return out
