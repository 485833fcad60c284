"""Host-side planning of a decode program (no GPU): the tiling the library chooses for the
operations of a step, and what it refuses."""
from __future__ import annotations

import pytest

from celeg_b200 import kernels

SMS, SMEM = 148, 232448          # a B200: SMs and opt-in shared memory per block


def product(rows, n, k, wt=1, epilogue=0, normed=True, **extra):
    op = kernels.ProgramOp()
    op.kind, op.rows, op.n, op.k, op.wt, op.epilogue = kernels.OP_GEMV, rows, n, k, wt, epilogue
    op.w, op.y, op.ldw, op.ldy, op.tile_offset = 0x10000, 0x20000, k, n, n
    if normed:
        op.x_source, op.residual, op.norm_weight, op.eps, op.ld_residual = kernels.X_NORM, 0x30000, 0x40000, 1e-5, k
    else:
        op.x_source, op.x, op.ldx, op.x_rows = kernels.X_GLOBAL, 0x50000, k, 64
    for name, value in extra.items():
        setattr(op, name, value)
    return op


def conv(rows, n, k):
    return product(rows, n, k, wt=3, epilogue=4, conv_w=0x60000, state=0x70000, span_slot=0x80000, taps=3)


def plan(ops):
    packed, layout = kernels.decode_program_prepare(ops, sms=SMS, smem_limit=SMEM)
    planned = (kernels.ProgramOp * len(ops)).from_buffer_copy(packed)
    return planned, layout


def test_layout_for_the_widths_of_a_1p2b_model():
    ops = [conv(8, 2048, 2048), product(8, 2048, 2048, epilogue=2, normed=False),
           product(8, 8192, 2048, wt=2, epilogue=3), product(8, 2048, 8192, epilogue=2, normed=False),
           product(8, 65536, 2048, epilogue=1)]
    planned, layout = plan(ops)
    assert layout.row_tiles == 1 and layout.grid == SMS
    assert layout.stages >= 4 and layout.smem_bytes <= SMEM
    assert layout.x_bytes >= 8 * (2048 * 2 + 64)
    for op in planned:
        assert op.kc % 256 == 0 and 256 <= op.kc
        per_box = op.wt * 16 * 512 + (0 if op.x_source == kernels.X_NORM else 8 * 512)
        assert op.kc // 256 * per_box <= layout.stage_bytes
    # chunks of even length: 8,192 in equal pieces
    assert 8192 % planned[3].kc == 0 or (8192 + planned[3].kc - 1) // planned[3].kc * planned[3].kc - 8192 < 256 * 2


def test_sixteen_rows_take_two_row_tiles_and_fewer_stages():
    _, eight = plan([product(8, 2048, 2048)])
    _, sixteen = plan([product(16, 2048, 2048)])
    assert (eight.row_tiles, sixteen.row_tiles) == (1, 2)
    assert sixteen.x_bytes == 2 * eight.x_bytes and sixteen.stages <= eight.stages
    assert sixteen.smem_bytes <= SMEM


def test_small_and_odd_sizes_are_taken():
    planned, layout = plan([product(3, 100, 72), product(3, 100, 136, epilogue=2, normed=False),
                            product(3, 777, 80, epilogue=1)])
    assert [op.kc for op in planned] == [256, 256, 256]
    assert layout.stages >= 3


@pytest.mark.parametrize("bad, words", [
    (dict(rows=17), "rows"),
    (dict(k=2052), "multiples of 8"),
    (dict(ldw=2044), "multiples of 8"),
    (dict(wt=2), "tile sets"),
    (dict(eps=0.0), "norm"),
    (dict(ldy=100), "ldy"),
])
def test_refusals_name_the_reason(bad, words):
    op = product(8, 2048, 2048)
    for name, value in bad.items():
        setattr(op, name, value)
    with pytest.raises(kernels.ProgramUnsupported, match=words):
        plan([op])


def test_a_width_that_leaves_no_room_for_stages_is_refused():
    with pytest.raises(kernels.ProgramUnsupported, match="shared memory"):
        plan([product(16, 4096, 8192)])          # the normalised operand alone would take 256 KiB


def test_attention_needs_its_buffers():
    op = kernels.ProgramOp()
    op.kind, op.rows, op.q_heads, op.kv_heads, op.head_dim = kernels.OP_ATTENTION, 4, 8, 2, 64
    with pytest.raises(kernels.ProgramUnsupported, match="lacks a buffer"):
        plan([op])
