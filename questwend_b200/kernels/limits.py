"""Sizes that the kernels take, as plain numbers: a configuration or a part can refuse what lies outside when a model
is put together, before a weight is read, instead of at its first step.  (The kernels check again at every launch.)"""

HEAD_DIM_STEP = 16          # attention takes head sizes that are multiples of this ...
MAX_HEAD_DIM = 256          # ... up to this (csrc/attention.cu: QWB_MAX_HEAD_DIM)


def head_dim_refusal(head_dim: int) -> str | None:
    """None if the attention kernels take this head size, else why not."""
    if head_dim <= 0 or head_dim % HEAD_DIM_STEP or head_dim > MAX_HEAD_DIM:
        return (f"the attention kernels take head sizes that are multiples of {HEAD_DIM_STEP} from {HEAD_DIM_STEP} to "
                f"{MAX_HEAD_DIM}, not {head_dim}")
    return None


CONV_MAX_TAPS = 16          # csrc/recurrent.cu: QWB_CONV_MAX_TAPS
SCAN_MAX_ROWS = 512         # rows of a recurrent state's column that one warp keeps in registers (csrc/recurrent.cu)
LATENT_MAX_RANK = 512       # csrc/attention_latent.cu: QWB_LATENT_MAX_L
LATENT_MAX_ROW = 1024       # ... QWB_LATENT_MAX_ROW
MOE_MAX_TOP = 16            # csrc/moe.cu: QWB_MOE_MAX_TOP


def conv_taps_refusal(taps: int) -> str | None:
    if not 1 <= taps <= CONV_MAX_TAPS:
        return f"the short convolution takes 1 to {CONV_MAX_TAPS} taps, not {taps}"
    return None


def state_matrix_refusal(rows: int, cols: int) -> str | None:
    """A recurrent state of rows x cols per head (state or key size x value size)."""
    if rows <= 0 or cols <= 0 or rows > SCAN_MAX_ROWS:
        return (f"the recurrence kernels keep a state of up to {SCAN_MAX_ROWS} rows (key or state size) per head, "
                f"not {rows} x {cols}")
    return None


def latent_refusal(rank: int, rot_dim: int) -> str | None:
    if rank <= 0 or rot_dim < 0 or rank > LATENT_MAX_RANK or rank + rot_dim > LATENT_MAX_ROW:
        return (f"the latent attention kernel takes a latent of up to {LATENT_MAX_RANK} values and a cached row of up to "
                f"{LATENT_MAX_ROW}, not {rank} + {rot_dim}")
    return None


def moe_refusal(experts: int, top: int) -> str | None:
    if experts <= 0 or not 1 <= top <= min(experts, MOE_MAX_TOP):
        return f"the router chooses 1 to {MOE_MAX_TOP} of its experts, not {top} of {experts}"
    return None


POOL_ATTN_DIM_STEP = 8      # the window-and-blocks attention takes key and value sizes that are multiples of this ...
POOL_ATTN_MAX_DIM = 256     # ... up to this (csrc/attention_pool.cu: QWB_POOL_MAX_DIM)


def pool_attention_refusal(dim: int, vdim: int) -> str | None:
    for what, n in (("key", dim), ("value", vdim)):
        if n <= 0 or n % POOL_ATTN_DIM_STEP or n > POOL_ATTN_MAX_DIM:
            return (f"the window-and-blocks attention takes {what} sizes that are multiples of {POOL_ATTN_DIM_STEP} up to "
                    f"{POOL_ATTN_MAX_DIM}, not {n}")
    return None


MAPS_ATTN_MAX_DIM = 256     # the attention with score maps takes key and value sizes up to this (csrc/attention_maps.cu:
MAPS_ATTN_MAX_MAPS = 2      # QWB_MAPS_MAX_DIM) and this many score maps per head (QWB_MAPS_MAX)
MAPS_ATTN_FAST_STEP = 8     # sizes that are multiples of this take the kernels that copy 16 bytes at a time; others the plain one


def maps_attention_refusal(maps: int, dim: int, vdim: int) -> str | None:
    if not 1 <= maps <= MAPS_ATTN_MAX_MAPS:
        return f"the attention with score maps takes 1 or {MAPS_ATTN_MAX_MAPS} maps per head, not {maps}"
    for what, n in (("key", dim), ("value", vdim)):
        if n <= 0 or n > MAPS_ATTN_MAX_DIM:
            return f"the attention with score maps takes {what} sizes up to {MAPS_ATTN_MAX_DIM}, not {n}"
    return None


SHAPED_ATTN_MAX_DIM = 256   # the attention with shaped scores takes key and value sizes up to this (csrc/attention_bias.cu:
                            # QWB_BIAS_MAX_DIM); sizes that are multiples of 8 take the kernels that copy 16 bytes at a time


def shaped_attention_refusal(dim: int, vdim: int) -> str | None:
    for what, n in (("key", dim), ("value", vdim)):
        if n <= 0 or n > SHAPED_ATTN_MAX_DIM:
            return f"the attention with shaped scores takes {what} sizes up to {SHAPED_ATTN_MAX_DIM}, not {n}"
    return None
