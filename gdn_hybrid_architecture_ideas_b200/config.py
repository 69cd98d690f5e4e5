"""Configuration: nested dataclasses, YAML round trip, dotted overrides and refuse-by-name checks.

The field names, nesting and defaults are the public configuration surface of the hybrid GDN/attention language
model family (reference: ced/config.py:25-2316), so run files and checkpoint configs written for it load here
unchanged. Options of experimental arms that this framework does not build are still *fields* (so a file naming
them at their default parses) but `unsupported_options` names every one that is set to a value with no
implementation, and `build_model` / `Trainer` refuse such a config with that list (reference rule: nothing is
silently ignored, ced/model/control.py:201-1243).

B200-specific additions live in `RuntimeConfig`-free form: they are plain keyword arguments of the engine
(`kernels=`, `parallel=`), never config keys, so a checkpoint's config stays readable by the reference.
"""

from __future__ import annotations

import ast
import dataclasses
import typing
from dataclasses import dataclass, field
from pathlib import Path

import yaml


class _Section:
    """Base of every config section: list values of tuple-typed fields become tuples (YAML and --set give lists),
    by-layer tables get integer keys, so two configs compare equal however they were written."""

    _TUPLE_FIELDS = frozenset({"nope_global_layers", "fused_projections", "keep_names", "fp8_names", "chains", "folds",
                               "recur_layers", "layers"})
    _TABLE_FIELDS = frozenset({"gdn_shape_by_layer", "heads_by_layer"})

    def __setattr__(self, name, value):
        if name in self._TUPLE_FIELDS and isinstance(value, list):
            value = tuple(value)
        elif name in self._TABLE_FIELDS and isinstance(value, dict):
            value = {(int(k) if isinstance(k, str) and k.isdigit() else k): (tuple(v) if isinstance(v, list) else v)
                     for k, v in value.items()}
        object.__setattr__(self, name, value)


@dataclass
class AttentionConfig(_Section):
    n_q_heads: int = 16
    n_kv_heads: int = 2
    head_dim: int = 256
    gate: str = 'elementwise'
    qk_norm: bool = True
    rope_fraction: float = 0.25
    rope_theta: float = 10000000.0
    rope_max_distance: int | None = None
    backend: str = 'reference'
    fa3_docs_per_row: int = 64
    fa4_deterministic: bool = True
    flex_tiles: str = 'classified'
    row_term: str = 'stored_o'
    temperature: str = 'fixed'
    temperature_ref_len: int = 8192
    normalizer: str = 'softmax'
    asentmax_chunk: int = 0
    kv_sharing: str = 'gqa'
    grid_rows: int = 0
    grid_cols: int = 0
    row_dim: int = 0
    col_dim: int = 0
    heads_per_cell: int = 1
    grid_depth: int = 0
    depth_dim: int = 0

@dataclass
class GDNNegEigConfig(_Section):
    beta_max: int = 1

@dataclass
class KDAConfig(_Section):
    decay: str = 'scalar'
    proj: str = 'shared'
    rank: int = 0
    floor_channels: int = 0
    floor_min: float = 64.0
    floor_max: float = 262144.0
    kernel: str = 'chunk_kda'

@dataclass
class EraseConfig(_Section):
    mode: str = 'none'
    rank: int = 16

@dataclass
class DeltaProductConfig(_Section):
    n_h: int = 1
    route: str = 'interleave'
    beta_max: int = 2
    beta_init: float | None = None
    layers: tuple = ()
    heads: int = 0
    heads_by_layer: dict = field(default_factory=dict)
    key: str = 'proj'
    value: str = 'proj'
    beta: str = 'proj'
    rank: int = 16
    perm: str = 'roll'
    conv: bool = True
    stride: int = 1
    summary: str = 'none'
    first_beta: str = 'carry'
    sparse_path: str | None = None

@dataclass
class GDNConfig(_Section):
    n_k_heads: int = 16
    n_v_heads: int = 16
    k_head_dim: int = 128
    v_head_dim: int = 128
    conv_kernel: int = 4
    init: str = 'fla'
    kernel: str = 'recurrence'
    chunk_size: int = 64
    output_gate: str = 'silu'
    input_dtype: str = 'float32'
    decay_cumsum: str = 'plain'
    edges: str = 'plain'
    chunk_backend: str = 'triton'
    negeig: GDNNegEigConfig = field(default_factory=GDNNegEigConfig)
    kda: KDAConfig = field(default_factory=KDAConfig)
    erase: EraseConfig = field(default_factory=EraseConfig)
    dprod: DeltaProductConfig = field(default_factory=DeltaProductConfig)

class _EncoderLayout:
    """Layer layout helpers of EncoderConfig (reference: ced/config.py:710-745)."""

    def layer_kinds(self) -> list[str]:
        """Kind of every layer, bottom first: layer i is softmax attention iff (i + 1) is a multiple of
        full_attn_interval, else Gated DeltaNet."""
        step = self.full_attn_interval
        return ["attention" if step > 0 and (i + 1) % step == 0 else "gdn" for i in range(self.n_layers)]

    def global_layers(self) -> list[int]:
        return [i for i, kind in enumerate(self.layer_kinds()) if kind == "attention"]

    def gdn_layers(self) -> list[int]:
        return [i for i, kind in enumerate(self.layer_kinds()) if kind == "gdn"]

    def nope_layers(self) -> tuple[int, ...]:
        """nope_global_layers validated: distinct ascending ordinals of global layers (0 = the lowest one)."""
        idx, n = self.nope_global_layers, len(self.global_layers())
        good = isinstance(idx, tuple) and all(type(i) is int and 0 <= i < n for i in idx) and list(idx) == sorted(set(idx))
        if not good:
            raise ValueError(f"model.encoder.nope_global_layers {idx!r}: ascending distinct ordinals among the {n} "
                             f"global attention layers (0 .. {n - 1})")
        return idx

    def gdn_shapes(self) -> list["GDNConfig"]:
        """GDNConfig of every GDN layer, bottom first. `gdn_shape_by_layer` {GDN ordinal: [n_k_heads, n_v_heads, head_dim]}
        gives a layer a copy of `gdn` with its own head counts and head size (key and value alike); without the table every
        entry is `gdn` itself (reference: ced/config.py:741-770)."""
        n = len(self.gdn_layers())
        table = self.gdn_shape_by_layer
        if not table:
            return [self.gdn] * n
        if not isinstance(table, dict):
            raise ValueError(f"model.encoder.gdn_shape_by_layer {table!r}: a mapping {{GDN ordinal: [n_k_heads, n_v_heads, head_dim]}}")
        bad = [k for k in table if type(k) is not int or not 0 <= k < n]
        if bad:
            raise ValueError(f"model.encoder.gdn_shape_by_layer keys {bad!r}: GDN ordinals among the encoder's {n} GDN layers (0 .. {n - 1})")
        out = []
        for i in range(n):
            if i not in table:
                out.append(self.gdn)
                continue
            shape = table[i]
            if not (isinstance(shape, (list, tuple)) and len(shape) == 3 and all(type(v) is int and v >= 1 for v in shape)):
                raise ValueError(f"model.encoder.gdn_shape_by_layer[{i}] {shape!r}: [n_k_heads, n_v_heads, head_dim], three integers >= 1")
            hk, hv, hd = shape
            if hv % hk:
                raise ValueError(f"model.encoder.gdn_shape_by_layer[{i}] {list(shape)!r}: n_v_heads must be a multiple of n_k_heads")
            out.append(dataclasses.replace(self.gdn, n_k_heads=hk, n_v_heads=hv, k_head_dim=hd, v_head_dim=hd))
        return out

    def dprod_carry(self) -> list:
        """Which value heads of each GDN layer carry Gated DeltaProduct's extra steps, bottom first. None for every layer at
        n_h 1 (the placement keys must then be at their defaults); else a tuple of value-head indices against the layer's
        own shape: () for a layer that does not carry, every head for one that carries as a whole, a union of whole key
        groups for one that carries some. `dprod.layers`: the GDN ordinals that carry (() = all); `dprod.heads` m: the
        first m value heads of a carrying layer (0 = all); `dprod.heads_by_layer` {ordinal: heads} wins over `heads`
        (reference: ced/config.py:775-834)."""
        d, shapes = self.gdn.dprod, self.gdn_shapes()
        n = len(shapes)
        used = [k for k, on in (("layers", d.layers != ()), ("heads", d.heads != 0), ("heads_by_layer", d.heads_by_layer != {})) if on]
        if d.n_h == 1:
            if used:
                raise ValueError(f"model.encoder.gdn.dprod.{', '.join(used)} set with n_h 1: the placement keys are read only with n_h >= 2")
            return [None] * n
        layers = tuple(d.layers) if isinstance(d.layers, (list, tuple)) else d.layers
        if not (isinstance(layers, tuple) and all(type(i) is int and 0 <= i < n for i in layers) and list(layers) == sorted(set(layers))):
            raise ValueError(f"model.encoder.gdn.dprod.layers {d.layers!r}: distinct GDN ordinals among the encoder's {n} GDN layers "
                             f"(0 .. {n - 1}) in ascending order, or () for every layer")
        if type(d.heads) is not int or d.heads < 0:
            raise ValueError(f"model.encoder.gdn.dprod.heads {d.heads!r}: an integer >= 0 (0: every value head of a carrying layer)")
        if not isinstance(d.heads_by_layer, dict):
            raise ValueError(f"model.encoder.gdn.dprod.heads_by_layer {d.heads_by_layer!r}: a mapping {{GDN ordinal: [value heads]}}")
        table = {int(k) if isinstance(k, str) and k.isdigit() else k: v for k, v in d.heads_by_layer.items()}
        carrying = set(layers) if layers else set(range(n))
        stray = [k for k in table if type(k) is not int or k not in carrying]
        if stray:
            raise ValueError(f"model.encoder.gdn.dprod.heads_by_layer keys {stray!r}: ordinals of layers that carry the extra steps ({sorted(carrying)!r})")
        out = []
        for i in range(n):
            if i not in carrying:
                out.append(())
                continue
            hk, hv = shapes[i].n_k_heads, shapes[i].n_v_heads
            g = hv // hk
            if i in table:
                heads = table[i]
                if not (isinstance(heads, (list, tuple)) and len(heads) > 0 and all(type(h) is int and 0 <= h < hv for h in heads)
                        and list(heads) == sorted(set(heads))):
                    raise ValueError(f"model.encoder.gdn.dprod.heads_by_layer[{i}] {heads!r}: distinct value heads among this layer's {hv} "
                                     f"(0 .. {hv - 1}) in ascending order, at least one")
                chosen = tuple(heads)
            elif d.heads:
                if d.heads % g or d.heads > hv:
                    raise ValueError(f"model.encoder.gdn.dprod.heads {d.heads}: a multiple of the layer's {g} value heads a key head and at "
                                     f"most its {hv} value heads (GDN layer {i})")
                chosen = tuple(range(d.heads))
            else:
                chosen = tuple(range(hv))
            cut = [k for k in sorted({h // g for h in chosen}) if not all(h in chosen for h in range(k * g, (k + 1) * g))]
            if cut:
                raise ValueError(f"model.encoder.gdn.dprod value heads {list(chosen)!r} of GDN layer {i}: key head(s) {cut!r} would be cut "
                                 f"(a key head serves {g} consecutive value heads; the rule takes whole key groups)")
            out.append(chosen)
        return out

    def gdn_layer_configs(self) -> list:
        """(GDNConfig, carrying heads or None) each GDN layer is built from: `gdn_shapes()` with the placement applied. A layer
        that does not carry gets the default DeltaProductConfig (n_h 1: the plain layer); one that carries gets the model's
        own with the placement keys reset; the heads are None where every head carries (reference: ced/config.py:836-850)."""
        shapes, carry, d = self.gdn_shapes(), self.dprod_carry(), self.gdn.dprod
        if d.n_h == 1 or (d.layers == () and d.heads == 0 and d.heads_by_layer == {}):
            return [(c, None) for c in shapes]
        own = dataclasses.replace(d, layers=(), heads=0, heads_by_layer={})
        return [(dataclasses.replace(c, dprod=own if h else DeltaProductConfig()), None if not h or len(h) == c.n_v_heads else tuple(h))
                for c, h in zip(shapes, carry)]

    def global_attention(self) -> list["AttentionConfig"]:
        """Attention config of each global layer, bottom first; a layer listed in nope_global_layers gets a copy with
        rope_fraction 0 and no distance cap (position-free attention)."""
        nope = set(self.nope_layers())
        return [dataclasses.replace(self.attention, rope_fraction=0.0, rope_max_distance=None) if g in nope
                else self.attention for g in range(len(self.global_layers()))]


@dataclass
class EncoderConfig(_Section, _EncoderLayout):
    n_layers: int = 36
    full_attn_interval: int = 4
    attention: AttentionConfig = field(default_factory=AttentionConfig)
    gdn: GDNConfig = field(default_factory=GDNConfig)
    loops: int = 1
    nope_global_layers: tuple[int, ...] = ()
    layer_scalars: str = 'none'
    layer_scalars_span: float = 4.0
    canon_kernel: int = 0
    canon_init: str = 'zeros'
    attn_res: str = 'none'
    attn_res_heads: int = 1
    attn_res_query: str = 'static'
    attn_res_query_hidden: int = 0
    attn_res_fused: bool = False
    ldm_groups: int = 8
    ldm_key_dim: int = 8
    ldm_hidden: int = 0
    block_norm_gain: str = 'channel'
    gdn_write_mix: str = 'none'
    gdn_write_variant: str = 'none'
    gdn_qmix_select_step: int = 0
    mix_fold: bool | str = False
    write_mix_storage: str = 'float32'
    write_mix_row_term: str = 'stored_o'
    residual_dtype: str = 'float32'
    gdn_ccr_spacing: int = 0
    gdn_ccr_target: str = 'previous'
    gdn_ccr_translator: str = 'none'
    gdn_ccr_gate_init: float = 0.0
    gdn_ccr_gate_floor: float = 0.0
    gdn_shape_by_layer: dict = field(default_factory=dict)

@dataclass
class DecoderConfig(_Section):
    n_layers: int = 4
    attention: AttentionConfig = field(default_factory=AttentionConfig)
    memory_attn_interval: int = 1
    gdn: GDNConfig = field(default_factory=GDNConfig)
    ffn_experts: int = 0
    ffn_top_k: int = 2
    ffn_expert_hidden: int | None = None
    moe_balance_weight: float = 0.01
    untie_mixers: str = 'none'
    router_z_weight: float = 0.0
    memory_kv_per_layer: bool = False
    capacity_fraction: float = 0.25
    capacity_multiple: int = 128
    self_kv: bool = False
    read_pattern: str = 'F'
    local_window: int = 128
    n_sinks: int = 4
    local_temperature: str = 'inherit'

    def layer_kinds(self) -> list[str]:
        """Every `memory_attn_interval`-th decoder layer reads the memory; the others are Gated DeltaNet over the slots."""
        every = self.memory_attn_interval
        return ["gdn" if (i + 1) % every else "memory_attention" for i in range(self.n_layers)]

@dataclass
class LoopConfig(_Section):
    t_max: int = 3
    t_choices: list[int] = field(default_factory=lambda: [3])
    t_probs: list[float] = field(default_factory=lambda: [1.0])
    t_eval: int = 3
    injection: str = 'parcae'
    parcae_init_decay: float = 0.4472135954999579
    loop_embedding: bool = True
    hyper_connections: str = 'none'
    draft_loss_weight: float = 0.0
    depth_attention: str = 'none'
    depth_attention_head_dim: int = 128
    depth_attention_rope_theta: float = 500.0
    hc_streams: int = 2
    hc_write: str = 'delta'
    hc_res_init: float = 0.05
    pass2_gate: str = 'none'
    segment_passes: dict | None = None
    segment_tokenizer: str | None = None
    unscored_passes: int | None = None
    pass2_layers: int = 0
    recur_layers: tuple[int, ...] = ()
    recur_inject_b: str = 'dense'
    recur_state_init: str = 'zeros'
    recur_prelude_norm: bool = True
    recur_mix_init: float = 0.99
    t_sampling: str = 'step'

@dataclass
class ResidualScaleConfig(_Section):
    mode: str = 'none'
    lam: float = 1.0
    depth_base: float = 1.0
    t_ref: int | None = None
    l_ref: float = 12.0

@dataclass
class SecondPassConfig(_Section):
    pass_embedding: bool = True

@dataclass
class NVFP4Config(_Section):
    mode: str = 'none'
    keep_last_fraction: float = 0.0
    keep_first_layers: int = 0
    stochastic_rounding: bool = True
    rht: bool = True
    weight_2d: bool = True
    keep_names: tuple[str, ...] = ()
    recipe: str = 'nvidia'
    fp8_names: tuple[str, ...] = ()
    until_step: int = 0

@dataclass
class FP8Config(_Section):
    mode: str = 'none'
    scaling: str = 'rowwise'
    backend: str = 'emulated'
    te_nonfinite_check: bool = False
    quantiser: str = 'torch'
    te_operands: str = 'te'
    nonfinite_flag: bool = False
    nonfinite_flag_form: str = 'pure'
    chains: tuple[str, ...] = ()
    folds: tuple[str, ...] = ()

@dataclass
class MTPConfig(_Section):
    enabled: bool = False
    block: str = 'attention'

@dataclass
class CPHeadConfig(_Section):
    enabled: bool = False
    d_c: int = 64
    query_chunk: int = 512
    force_lambda_zero: bool = False
    score: str = 'mixture'
    train_mode: str = 'mixture'
    aux_weight: float = 0.0
    qk_norm: bool = False
    init: str = 'spec'
    kernel: str = 'reference'
    window: int = 0
    pointer_input: str = 'final'
    shared_layer: int = -1
    shared_head: int = 0
    shared_ssmax: bool = False
    temperature: str = 'none'
    sink_count: bool = False
    n_heads: int = 1
    combine: str = 'and'
    trunk_copy: str = 'none'
    trunk_k: int = 0
    trunk_select_step: int = 0

@dataclass
class ModelConfig(_Section):
    arch: str = 'looped_ced'
    vocab_size: int = 128000
    tie_embeddings: bool = True
    d_model: int = 2560
    ffn_hidden: int = 7168
    ffn_activation: str = 'swiglu'
    norm_eps: float = 1e-06
    embed_norm: bool = True
    init_std: float = 0.02
    encoder: EncoderConfig = field(default_factory=EncoderConfig)
    decoder: DecoderConfig = field(default_factory=DecoderConfig)
    loop: LoopConfig = field(default_factory=LoopConfig)
    residual_scale: ResidualScaleConfig = field(default_factory=ResidualScaleConfig)
    second_pass: SecondPassConfig = field(default_factory=SecondPassConfig)
    nvfp4: NVFP4Config = field(default_factory=NVFP4Config)
    fp8: FP8Config = field(default_factory=FP8Config)
    mtp: MTPConfig = field(default_factory=MTPConfig)
    cp_head: CPHeadConfig = field(default_factory=CPHeadConfig)
    fused_projections: tuple[str, ...] = ()

@dataclass
class DataConfig(_Section):
    kind: str = 'synthetic'
    shard_dir: str | None = None
    extra_shard_dirs: list[str] = field(default_factory=list)
    union_order: str = 'permute'
    span_fraction: float = 0.25
    seq_len: int = 64
    batch_size: int = 2
    doc_len_min: int = 8
    doc_len_max: int = 40
    span_distribution: str = 'lognormal'
    span_median: float = 230.0
    span_sigma: float = 1.16
    span_min: int = 16
    span_max: int = 4096
    seed: int = 1234
    chat_whole: bool = False
    fit_decoder_capacity: bool = False
    decoder_positions: str = 'data'
    answer_min_context: int = 1024
    answer_gap_mean: float = 1024.0
    answer_capacity_fraction: float = 1.0
    answer_sinks: bool = True
    answer_replay_window: int = 0
    loss_mask: str = 'all'

@dataclass
class OursConfig(_Section):
    m1: bool = False
    m1_theta: float = 0.0
    m2: bool = False
    m2_beta: float = 0.0
    m2_memory: float = 0.08
    m2_alpha: float = 5.0
    m2_warmup: int = 0
    m3: bool = False
    m3_p: float = 0.25
    m3_k: int = 16
    m3_every: int = 20
    m3_beta: float = 0.95
    m3_cmin: float = 0.1
    m3_snr: bool = False
    m4: bool = False
    m4_reset_fast: bool = True
    m4_layers: int = 4
    log_every: int = 0
    rotation_log_every: int = 0
    lite_chi: float = 2.0
    lite_ratio: float = 0.1
    samuon_gamma: float = 7.07
    samuon_warmup: float = 0.3
    samuon_iters: int = 10

@dataclass
class OptimConfig(_Section):
    name: str = 'adamw'
    lr: float = 0.003
    betas: list[float] = field(default_factory=lambda: [0.9, 0.95])
    eps: float = 1e-08
    weight_decay: float = 0.1
    grad_clip: float = 1.0
    warmup_steps: int = 10
    decay_fraction: float = 0.2
    muon_momentum: float = 0.95
    muon_nesterov: bool = True
    muon_ns_steps: int = 5
    adamw_lr_scale: float = 1.0
    pass2_lr_scale: float = 1.0
    schedule_steps: int | None = None
    layer_scalar_a_lr_scale: float = 1.0
    recur_b: str = 'adamw'
    switch_warmup_steps: int = 0
    hyperball: bool = False
    hyperball_radius: float = 0.0
    soap_shampoo_beta: float = 0.95
    soap_precondition_frequency: int = 1
    soap_eigh: bool = False
    shampoo_epsilon: float = 1e-12
    shampoo_precondition_frequency: int = 100
    shampoo_start_step: int = -1
    normuon_beta2: float = 0.95
    gdn_mup: bool = False
    gdn_mup_base_width: int = 512
    zero_gate_decay: str = 'decay'
    mix_query_decay: str = 'decay'
    ccr_translator_decay: str = 'none'
    anvil2_preset: str = 'style'
    anvil2_single_rounding: bool = False
    anvil2_tavg: bool = False
    anvil2_decon: str = 'matrix'
    anvil2_scale: str = 'ours'
    anvil2_points: str | None = None
    anvil2_tail_ema: bool = False
    anvil2_qk_head_pairs: bool = False
    lr_floor: float = 0.0
    soap_seeded_start: bool = False
    ours: OursConfig = field(default_factory=OursConfig)

@dataclass
class LossConfig(_Section):
    aux_weight: float = 1.0
    z_loss: float = 0.0001
    normalization: str = 'global_token_mean'
    aux_positions: str = 'context'
    aux_fraction: float = 0.5
    ce_form: str = 'standard'

@dataclass
class WandbConfig(_Section):
    mode: str = 'disabled'
    project: str = 'looped-ced'
    entity: str | None = None
    run_name: str | None = None

@dataclass
class EvalConfig(_Section):
    sets: dict = field(default_factory=dict)
    every_steps: int = 0
    periodic_max_rows: int = 64
    batch_size: int = 1
    replay_window: int | str = 128
    decoder_at: str | None = None
    lc_every_steps: int = 0
    lc_dir: str | None = None
    lc_length: int = 0
    lc_docs: int = 12
    lc_base_len: int = 8192
    lc_mf_items: int = 0
    readout_every: int = 0
    readout_sets: list = field(default_factory=list)
    readout_batch_tokens: int = 16384
    bpb_readout_every: int = 0
    bpb_readout_from: int = 0
    bpb_readout_sets: dict = field(default_factory=dict)
    bpb_readout_rows: int = 256
    bpb_readout_seed: int = 0

@dataclass
class TSTConfig(_Section):
    schedule: list = field(default_factory=list)
    gdn_decay_rescale: bool = False
    token_scale_rope: bool = False
    phase1_exclude_sources: list = field(default_factory=list)
    aux_multi_hot: int = 0
    aux_weight: float = 0.1
    gdn_resolution_gates: str = 'none'
    gdn_conv_reinit: bool = False
    bag_lr_power: float = 0.0
    rewarm_steps: int = 0
    output_only: bool = False
    bag_input: str = 'mean'
    keep_optimizer_state: bool = False

@dataclass
class TrainConfig(_Section):
    model: ModelConfig = field(default_factory=ModelConfig)
    data: DataConfig = field(default_factory=DataConfig)
    optim: OptimConfig = field(default_factory=OptimConfig)
    loss: LossConfig = field(default_factory=LossConfig)
    wandb: WandbConfig = field(default_factory=WandbConfig)
    eval: EvalConfig = field(default_factory=EvalConfig)
    steps: int = 100
    seed: int = 0
    dtype: str = 'float32'
    log_every: int = 10
    ckpt_every_steps: int = 50
    ckpt_every_minutes: float = 7.5
    ckpt_keep: int = 3
    ckpt_async: bool = False
    data_prefetch: bool = False
    device: str = 'auto'
    autocast: str = 'none'
    micro_batch_size: int | None = None
    tf32: bool = False
    deterministic: bool = False
    fill_uninitialized_memory: bool = True
    metrics_jsonl: bool = False
    compile: str = 'none'
    head_select: bool = False
    head_impl: str = 'chunked'
    head_precision: str = 'fp32'
    head_chunk: int = 2048
    trim_decoder_slots: int = 0
    decoder_opt: str = 'none'
    activation_checkpoint: str = 'none'
    init_from: str | None = None
    freeze_trunk: bool = False
    checkpoint_steps: list[int] = field(default_factory=list)
    resume_from: str | None = None
    loop_switch_step: int = 0
    stage: str = 'none'
    precision_switch: bool = False
    data_start_step: int = 0
    pass_slot_buckets: list[float] = field(default_factory=lambda: [1.0, 0.5, 0.25, 0.125, 0.0625])
    shape_schedule: list = field(default_factory=list)
    shape_lr: str = 'clock'
    micro_batch_by_t: list[int] = field(default_factory=list)
    log_stream_rms_every: int = 0
    log_zero_wgrad_every: int = 0
    cuda_graphs: str = 'none'
    cuda_graphs_docs_per_row: int = 64
    wgrad_accum: str = 'autograd'
    optimizer_sharding: str = 'replicated'
    tensor_parallel: int = 1
    tst: TSTConfig = field(default_factory=TSTConfig)
    stage_shape: str = 'source'



# ----------------------------------------------------------------------------------------------------------------
# dict / YAML round trip, dotted overrides
# ----------------------------------------------------------------------------------------------------------------


# Keys this framework adds to the reference's config tree. They are left out of a written dict while at their defaults, so
# a config or checkpoint of a run that does not use them loads, strictly, into the reference's dataclasses too.
EXTENSION_DEFAULTS = {"tensor_parallel": 1}


def to_dict(cfg) -> dict:
    out = dataclasses.asdict(cfg)
    if isinstance(cfg, TrainConfig):
        for key, default in EXTENSION_DEFAULTS.items():
            if out.get(key) == default:
                del out[key]
    return out


def from_dict(cls, data: dict | None):
    """Dataclass `cls` from a possibly partial nested dict; a key the section does not have raises KeyError
    (reference: ced/config.py:2328-2344)."""
    if data is None:
        return cls()
    hints = typing.get_type_hints(cls)
    names = {f.name for f in dataclasses.fields(cls)}
    extra = sorted(set(data) - names)
    if extra:
        raise KeyError(f"unknown keys for {cls.__name__}: {extra}")
    built = {}
    for key, value in data.items():
        section = hints[key]
        built[key] = from_dict(section, value) if dataclasses.is_dataclass(section) and isinstance(value, dict) else value
    return cls(**built)


def checkpoint_config(data: dict) -> dict:
    """A checkpoint's config dict as read today: model.fp8.nonfinite_flag_form defaults to "ordered" for files written
    before that key existed (reference: ced/config.py:2347-2355). Returns a new dict."""
    fp8 = (data.get("model") or {}).get("fp8")
    if not isinstance(fp8, dict) or "nonfinite_flag_form" in fp8:
        return data
    return {**data, "model": {**data["model"], "fp8": {**fp8, "nonfinite_flag_form": "ordered"}}}


def load_yaml(path: str | Path, cls=None):
    with open(path) as f:
        return from_dict(cls or TrainConfig, yaml.safe_load(f))


def save_yaml(cfg, path: str | Path) -> None:
    with open(path, "w") as f:
        yaml.safe_dump(to_dict(cfg), f, sort_keys=False)


def parse_value(text: str):
    """The value of a `--set key=value` override: a Python/YAML literal where it parses, else the string."""
    low = text.strip()
    if low in ("null", "None", "~"):
        return None
    if low in ("true", "True"):
        return True
    if low in ("false", "False"):
        return False
    try:
        return ast.literal_eval(low)
    except (ValueError, SyntaxError):
        return yaml.safe_load(low) if low[:1] in "[{" else low


def apply_override(cfg, assignment: str) -> None:
    """`a.b.c=value` applied to a config in place (reference: scripts/train.py:176-190). An unknown key raises
    KeyError naming the full path."""
    if "=" not in assignment:
        raise ValueError(f"override {assignment!r}: expected KEY=VALUE")
    path, raw = assignment.split("=", 1)
    node, parts = cfg, path.strip().split(".")
    for part in parts[:-1]:
        if not hasattr(node, part):
            raise KeyError(f"unknown config key {path!r} (no section {part!r})")
        node = getattr(node, part)
    leaf = parts[-1]
    if isinstance(node, dict):
        node[leaf] = parse_value(raw)
        return
    if not hasattr(node, leaf):
        raise KeyError(f"unknown config key {path!r}")
    setattr(node, leaf, parse_value(raw))


# ----------------------------------------------------------------------------------------------------------------
# refuse by name
# ----------------------------------------------------------------------------------------------------------------

_BUILT = {
    "model.arch": ("control", "looped_ced"),
    "model.ffn_activation": ("swiglu", "relu2"),
    "model.encoder.attention.gate": ("elementwise", "headwise", "none"),
    "model.encoder.attention.temperature": ("fixed", "learned", "ssmax"),
    "model.encoder.attention.normalizer": ("softmax", "asentmax"),
    "model.encoder.attention.kv_sharing": ("gqa", "grid"),
    "model.encoder.attention.row_term": ("stored_o",),
    "model.encoder.gdn.init": ("fla", "hf"),
    "model.encoder.gdn.output_gate": ("silu", "sigmoid"),
    "model.encoder.gdn.decay_cumsum": ("plain",),
    "model.encoder.gdn.kda.decay": ("scalar", "channel"),
    "model.encoder.gdn.erase.mode": ("none", "eda"),
    "model.encoder.gdn.negeig.beta_max": (1, 2),
    "model.encoder.gdn.dprod.n_h": (1, 2, 3, 4),
    "model.encoder.loops": (1,),
    "model.encoder.layer_scalars": ("none", "skip_x0", "skip_x0_span", "x0", "skip"),
    "model.encoder.attn_res": ("none", "block_entry", "block", "ldm"),
    "model.encoder.block_norm_gain": ("channel", "scalar"),
    "model.encoder.gdn_write_mix": ("none", "layer", "head"),
    "model.encoder.gdn_write_variant": ("none", "qmix", "korig", "vonly", "kqmix", "qshare", "qshare_kv", "qshare_bd"),
    "model.encoder.residual_dtype": ("float32", "bf16"),
    "model.loop.pass2_gate": ("none", "scalar"),
    "model.mtp.enabled": (False, True),
    "model.fp8.mode": ("none", "linears"),
    "model.fp8.scaling": ("rowwise", "tensorwise", "mxfp8"),
    "model.fp8.chains": ((),),
    "model.fp8.folds": ((),),
    "model.nvfp4.mode": ("none", "all_linears", "all_but_gdn", "all_but_gdn_mixer", "mlp_only"),
    "model.nvfp4.recipe": ("nvidia", "quartet2"),
}

_TRAIN_BUILT = {
    "optim.name": ("adamw", "muon"),
    "optim.hyperball": (False,),
    "optim.gdn_mup": (False, True),
    "loss.normalization": ("global_token_mean", "per_head_mean"),
    "loss.ce_form": ("standard", "fixed"),
    "head_impl": ("fused", "chunked"),
    "head_precision": ("fp32", "bf16"),
    "activation_checkpoint": ("none", "layer", "block", "host", "host_overlap"),
    "precision_switch": (False, True),
    "cuda_graphs": ("none", "microbatch"),        # "step" (clip + optimizer inside a graph) is not built: the update kernels take the LR by value
    "wgrad_accum": ("autograd", "fp32"),
    "optimizer_sharding": ("replicated", "zero1", "zero2"),
    "data.kind": ("synthetic", "shards", "uniform"),
    # the packer's fit of a row's assistant tokens to a decoder capacity belongs to the CED decoder, which is not built;
    # the span_* keys, span_fraction and decoder_positions only place that decoder's positions and are read by nothing here
    # (the control models train on every valid target), chat_whole is built (data/shards.py)
    "data.fit_decoder_capacity": (False,),
    "data.decoder_positions": ("data", "random"),
    "data.union_order": ("permute", "sets_in_order"),
    "decoder_opt": ("none",),
}


# Keys that belong to parts this framework does not build (the slot decoder of the looped architecture and its lane
# hyper-connections, the other matrix optimizers, the unbuilt forms of the Copy-Paste head, auxiliary losses, the in-loop
# long-context reads) and that nothing here reads. They load and round-trip; a value off the default would change nothing,
# so it is refused by name instead of being ignored.
_UNREAD = (
    "model.encoder.write_mix_storage", "model.encoder.write_mix_row_term", "model.decoder.self_kv", "model.decoder.read_pattern",
    "model.decoder.local_window", "model.decoder.local_temperature", "model.loop.hc_res_init", "model.second_pass.pass_embedding",
    "model.fp8.te_nonfinite_check", "model.fp8.te_operands", "model.fp8.nonfinite_flag", "model.fp8.nonfinite_flag_form",
    "model.cp_head.trunk_k",
    "model.cp_head.trunk_select_step")
# The slot decoder's keys: read by arch 'looped_ced' (models/looped_decoder.py), by nothing on the hybrid stack.
_UNREAD_STACK = (
    "model.decoder.memory_attn_interval", "model.decoder.ffn_experts", "model.decoder.ffn_top_k", "model.decoder.ffn_expert_hidden",
    "model.decoder.moe_balance_weight", "model.decoder.untie_mixers", "model.decoder.router_z_weight", "model.decoder.memory_kv_per_layer",
    "model.decoder.capacity_fraction", "model.decoder.capacity_multiple", "model.loop.draft_loss_weight", "model.loop.depth_attention",
    "model.loop.depth_attention_head_dim", "model.loop.depth_attention_rope_theta", "model.loop.hc_streams", "model.loop.hc_write")
_TRAIN_UNREAD = (
    "data.answer_min_context", "data.answer_gap_mean", "data.answer_capacity_fraction",
    "data.answer_sinks", "data.answer_replay_window", "optim.hyperball_radius", "optim.soap_shampoo_beta", "optim.soap_precondition_frequency",
    "optim.soap_eigh", "optim.shampoo_epsilon", "optim.shampoo_precondition_frequency", "optim.shampoo_start_step", "optim.normuon_beta2",
    "optim.anvil2_preset", "optim.anvil2_single_rounding", "optim.anvil2_tavg", "optim.anvil2_decon", "optim.anvil2_scale", "optim.anvil2_points",
    "optim.anvil2_tail_ema", "optim.anvil2_qk_head_pairs", "optim.soap_seeded_start", "optim.ours", "loss.aux_positions",
    "loss.aux_fraction", "eval.replay_window", "eval.decoder_at", "eval.lc_every_steps", "eval.lc_dir", "eval.lc_length", "eval.lc_docs",
    "eval.lc_base_len", "eval.lc_mf_items", "trim_decoder_slots", "pass_slot_buckets", "tst.aux_weight", "stage_shape")


def _get(cfg, dotted: str):
    node = cfg
    for part in dotted.split("."):
        node = getattr(node, part)
    return node


def unsupported_options(cfg) -> list[str]:
    """Every option of `cfg` (a ModelConfig or TrainConfig) set to a value this framework has no implementation
    for, as `key=value (built: ...)` strings. Empty list: the config can be built."""
    model = cfg.model if isinstance(cfg, TrainConfig) else cfg
    bad = []
    for key, allowed in _BUILT.items():
        value = _get(model, key[len("model."):])
        if value not in allowed:
            bad.append(f"{key}={value!r} (built: {list(allowed)})")
    if isinstance(cfg, TrainConfig):
        for key, allowed in _TRAIN_BUILT.items():
            value = _get(cfg, key)
            if value not in allowed:
                bad.append(f"{key}={value!r} (built: {list(allowed)})")
    plain_model, plain_train = ModelConfig(), TrainConfig()
    if isinstance(cfg, TrainConfig) and model.arch != "looped_ced":       # the two heads' loss keys: the hybrid stack has one head
        if cfg.loss.aux_weight != plain_train.loss.aux_weight or cfg.loss.normalization != plain_train.loss.normalization:
            bad.append(f"loss.aux_weight={cfg.loss.aux_weight!r} / loss.normalization={cfg.loss.normalization!r} (the two heads' loss of arch 'looped_ced'; read by nothing on arch {model.arch!r})")
    for key in _UNREAD + (_UNREAD_STACK if model.arch != "looped_ced" else ()):
        value, default = _get(model, key[len("model."):]), _get(plain_model, key[len("model."):])
        if value != default:
            bad.append(f"{key}={value!r} (read by nothing here: leave it {default!r})")
    if isinstance(cfg, TrainConfig):
        for key in _TRAIN_UNREAD:
            value, default = _get(cfg, key), _get(plain_train, key)
            if value != default:
                bad.append(f"{key}={value!r} (read by nothing here: leave it {default!r})")
    enc = model.encoder
    if enc.gdn_write_variant != "none" and enc.gdn_write_mix != "layer":
        bad.append("model.encoder.gdn_write_variant needs model.encoder.gdn_write_mix=layer")
    if enc.gdn_write_mix != "none" and enc.attn_res != "block_entry":
        bad.append("model.encoder.gdn_write_mix reads the finished blocks of model.encoder.attn_res=block_entry")
    if enc.attn_res_fused or enc.mix_fold:
        pass  # implementation switches of the reference's own fused kernels: accepted and ignored as IMPLEMENTATION_FIELDS
    if model.fp8.mode != "none" and model.nvfp4.mode != "none":
        bad.append("model.fp8.mode and model.nvfp4.mode are both set: one low-precision recipe at a time")
    return bad


def require_supported(cfg) -> None:
    bad = unsupported_options(cfg)
    if bad:
        raise ValueError("config options without an implementation in this framework: " + "; ".join(bad))


# Fields that select an implementation, not a model: two configs that differ only here describe the same training
# run, so a resume accepts the difference (reference: ced/train/trainer.py:592).
IMPLEMENTATION_FIELDS = (
    "model.encoder.attention.backend", "model.encoder.attention.flex_tiles", "model.encoder.attention.fa3_docs_per_row",
    "model.encoder.attention.fa4_deterministic", "model.encoder.attention.asentmax_chunk", "model.encoder.gdn.kernel", "model.encoder.gdn.edges",
    "model.encoder.gdn.chunk_backend", "model.encoder.attn_res_fused", "model.encoder.mix_fold",
    "model.decoder.attention.backend", "model.decoder.gdn.kernel", "model.fused_projections",
    "compile", "cuda_graphs", "cuda_graphs_docs_per_row", "head_impl", "head_chunk", "data_prefetch", "ckpt_async",
    "activation_checkpoint", "wgrad_accum", "device", "log_every", "metrics_jsonl", "ckpt_every_steps",
    "ckpt_every_minutes", "ckpt_keep", "checkpoint_steps", "steps", "wandb", "eval", "log_stream_rms_every",
    "log_zero_wgrad_every", "micro_batch_size", "optimizer_sharding", "deterministic", "fill_uninitialized_memory",
)


def config_differences(a: dict, b: dict, prefix: str = "") -> list[str]:
    """Dotted keys at which two config dicts differ, IMPLEMENTATION_FIELDS left out."""
    out = []
    for key in sorted(set(a) | set(b)):
        dotted = f"{prefix}{key}"
        if dotted in IMPLEMENTATION_FIELDS:
            continue
        va, vb = a.get(key), b.get(key)
        if isinstance(va, dict) and isinstance(vb, dict):
            out += config_differences(va, vb, dotted + ".")
        elif _plain(va) != _plain(vb):
            out.append(dotted)
    return out


def _plain(v):
    if isinstance(v, (list, tuple)):
        return [_plain(x) for x in v]
    return v


# ----------------------------------------------------------------------------------------------------------------
# presets
# ----------------------------------------------------------------------------------------------------------------


def tiny_data_config(**overrides) -> DataConfig:
    cfg = DataConfig(seq_len=64, batch_size=4, span_median=5.0, span_min=2, span_max=12)
    for key, value in overrides.items():
        setattr(cfg, key, value)
    return cfg


def tiny_control_config() -> ModelConfig:
    """CPU-sized plain hybrid stack: 10 layers, GDN/GDN/GDN/attention pattern, d_model 64
    (reference: ced/config.py:2373-2410)."""
    attn = AttentionConfig(n_q_heads=4, n_kv_heads=2, head_dim=16, rope_theta=1e4)
    gdn = GDNConfig(n_k_heads=2, n_v_heads=4, k_head_dim=16, v_head_dim=16, conv_kernel=4)
    return ModelConfig(arch="control", vocab_size=256, d_model=64, ffn_hidden=192,
                       encoder=EncoderConfig(n_layers=10, full_attn_interval=4, attention=attn, gdn=gdn))


def tiny_looped_config() -> ModelConfig:
    """CPU-sized looped encoder-decoder: 8 encoder layers, a 2-layer decoder block (GDN, memory attention) at up to 3 passes,
    a quarter of each row's positions in decoder slots."""
    cfg = tiny_control_config()
    cfg.arch = "looped_ced"
    cfg.encoder.n_layers = 8
    dec = cfg.decoder
    dec.n_layers, dec.memory_attn_interval, dec.capacity_fraction, dec.capacity_multiple = 2, 2, 0.25, 8
    dec.attention, dec.gdn = dataclasses.replace(cfg.encoder.attention), dataclasses.replace(cfg.encoder.gdn)
    cfg.loop.t_max, cfg.loop.t_choices, cfg.loop.t_probs, cfg.loop.t_eval = 3, [2, 3], [0.5, 0.5], 3
    return cfg


def tiny_full_config() -> ModelConfig:
    """CPU-sized model with every core feature on: block-entry depth mixing, qmix write/query mixes, distance cap,
    one position-free global layer, ssmax temperature, tied embeddings, v_head_dim != k_head_dim."""
    cfg = tiny_control_config()
    cfg.tie_embeddings = True
    enc = cfg.encoder
    enc.n_layers = 12
    enc.gdn = GDNConfig(n_k_heads=2, n_v_heads=4, k_head_dim=16, v_head_dim=32, conv_kernel=4, output_gate="sigmoid",
                        kernel="chunked", chunk_size=16)
    enc.attention.rope_max_distance = 24
    enc.attention.temperature = "ssmax"
    enc.attention.temperature_ref_len = 64
    enc.nope_global_layers = (2,)
    enc.attn_res = "block_entry"
    enc.gdn_write_mix = "layer"
    enc.gdn_write_variant = "qmix"
    return cfg


def hybrid_model_config(size: str, *, full: bool = True, kv: str = "gqa") -> ModelConfig:
    """The benchmark family: "60m" (d 512, 12 layers), "200m" (d 1024, 16 layers), "1p3b" (d 2048, 24 layers);
    3:1 GDN:attention, GDN key dim 128 / value dim 256, attention head_dim 64 with a 2048-token rotary distance cap
    and the last global layer position-free, SwiGLU, tied embeddings, vocabulary 32768. full: block-entry depth
    mixing and the qmix write/query mixes. kv "grid": 4 x 4 grid KV sharing (16 query heads) in place of GQA."""
    shapes = {"60m": (512, 12, 4, 8, 2, 1408), "200m": (1024, 16, 8, 16, 4, 2816), "1p3b": (2048, 24, 16, 32, 8, 5632)}
    d, layers, gdn_heads, hq, hkv, ffn = shapes[size]
    attn = AttentionConfig(n_q_heads=hq, n_kv_heads=hkv, head_dim=64, rope_fraction=0.25, rope_theta=1e7,
                           rope_max_distance=2048, gate="elementwise", qk_norm=True, backend="b200")
    if kv == "grid":
        assert hq == 16, "the 4 x 4 grid serves 16 query heads"
        attn.kv_sharing, attn.n_kv_heads = "grid", 1
        attn.grid_rows = attn.grid_cols = 4
        attn.row_dim = attn.col_dim = 32
    gdn = GDNConfig(n_k_heads=gdn_heads, n_v_heads=gdn_heads, k_head_dim=128, v_head_dim=256, conv_kernel=4,
                    output_gate="sigmoid", kernel="b200", chunk_size=64, input_dtype="bfloat16")
    enc = EncoderConfig(n_layers=layers, full_attn_interval=4, attention=attn, gdn=gdn)
    enc.nope_global_layers = (layers // 4 - 1,)
    if full:
        enc.attn_res, enc.gdn_write_mix, enc.gdn_write_variant = "block_entry", "layer", "qmix"
    return ModelConfig(arch="control", vocab_size=32768, tie_embeddings=True, d_model=d, ffn_hidden=ffn,
                       init_std=0.02, encoder=enc)
