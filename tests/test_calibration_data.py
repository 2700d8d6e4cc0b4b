"""Calibration-data generation (scripts/sample_diffusion_ddim.py:463-536): which (x_t, t) pairs
of a sampling run are kept, and the end-to-end generator on the device."""
import pytest
import torch

import cases


def _reference_selection(xs, ts, interval, cali_st, residual):
    """The reference's loop, statement for statement (scripts/sample_diffusion_ddim.py:492-504),
    as the checker of select_calibration_points."""
    xs_lst = [[] for _ in range(cali_st)]
    ts_lst = [[] for _ in range(cali_st)]
    xp_lst = [[] for _ in range(cali_st)]
    tp_lst = [[] for _ in range(cali_st)]
    for t in range(len(ts)):
        if t % interval == 0:
            xs_lst[t // interval].append(xs[t])
            ts_lst[t // interval].append(ts[t])
            if residual:
                if t <= 1:
                    xp_lst[t // interval].append(xs[t])
                    tp_lst[t // interval].append(ts[t])
                else:
                    xp_lst[t // interval].append(xs[t - 1])
                    tp_lst[t // interval].append(ts[t - 1])
    return xs_lst, ts_lst, xp_lst, tp_lst


@pytest.mark.parametrize("steps,cali_st,residual", [(20, 5, False), (20, 20, True), (12, 4, True)])
def test_selection_rule(steps, cali_st, residual):
    from modiff_b200.calibration import select_calibration_points
    xs = [torch.full((2, 1), float(i)) for i in range(steps + 1)]     # x_T .. x_0
    ts = [torch.full((2,), float(100 - i)) for i in range(steps)]
    interval = steps // cali_st
    got = select_calibration_points(xs, ts, interval, cali_st, residual)
    want = _reference_selection(xs, ts, interval, cali_st, residual)
    assert len(got) == cali_st
    for slot in range(cali_st):
        assert len(got[slot]) == len(want[0][slot]) == 1
        e = got[slot][0]
        assert torch.equal(e[0], want[0][slot][0]) and torch.equal(e[1], want[1][slot][0])
        if residual:
            assert torch.equal(e[2], want[2][slot][0]) and torch.equal(e[3], want[3][slot][0])
    with pytest.raises(ValueError):
        select_calibration_points(xs, ts, 3, 2, residual)          # 20 steps do not fit 2 x 3


@pytest.mark.gpu
def test_generate_on_the_device(cuda):
    """Two rounds of four images, 10 steps, 5 kept: shapes as the reference stacks them, the
    first slot is the noise itself, every kept state equals the state a plain sampling run of the
    same model enters that step with, and `residual` adds the previous step's pair."""
    import modiff_b200 as m
    torch.manual_seed(0)
    net = m.Model(m.make_config(split_shortcut=False)).to(cuda).eval()
    betas = torch.from_numpy(m.get_beta_schedule()).float()
    xs, ts, xp, tp = m.generate_calibration_data(net, (3, 32, 32), betas, timesteps=10, cali_n=7,
                                                 cali_st=5, batch_size=4, seed=11, residual=True,
                                                 device=cuda)
    assert tuple(xs.shape) == (5, 8, 3, 32, 32) and tuple(ts.shape) == (5, 8)
    assert tuple(xp.shape) == tuple(xs.shape) and tuple(tp.shape) == tuple(ts.shape)
    g = torch.Generator().manual_seed(11)
    x0 = torch.randn(4, 3, 32, 32, generator=g)
    assert torch.equal(xs[0, :4], x0)
    seq = m.make_timestep_sequence(1000, 10, "quad")
    run, tt, _ = m.generalized_steps(x0.to(cuda), seq, net, betas, with_t=True, last_only=False,
                                     eta=0.0)
    for slot in range(5):
        assert torch.equal(xs[slot, :4], run[2 * slot].cpu())
        assert torch.equal(ts[slot, :4], tt[2 * slot].cpu())
        prev = 2 * slot if 2 * slot <= 1 else 2 * slot - 1
        assert torch.equal(xp[slot, :4], run[prev].cpu())
    assert float(ts[0, 0]) == float(seq[-1]) and float(ts[-1, 0]) == float(seq[1])
