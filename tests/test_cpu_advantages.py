"""PPO advantage helpers against plain Python loops: KL-shaped rewards, GAE over ragged masks (padding on either side
and holes), whitening, the clipped value loss, and one PPO-clip step through the registry's ``ppo_loss``."""

import torch

from rl_engine.alignment import gae_advantages, kl_shaped_rewards, value_loss, whiten


def _inputs(seed=0, b=4, t=7):
    gen = torch.Generator().manual_seed(seed)
    mask = torch.ones(b, t, dtype=torch.bool)
    mask[1, 4:] = False            # right padding
    mask[2, :3] = False            # left padding
    mask[3, 2] = False             # a hole
    return gen, mask


def test_gae_matches_a_per_row_loop_over_the_real_tokens():
    gen, mask = _inputs()
    rewards, values = torch.randn(4, 7, generator=gen), torch.randn(4, 7, generator=gen)
    gamma, lam = 0.97, 0.9
    adv, ret = gae_advantages(rewards, values, mask, gamma=gamma, lam=lam)
    for row in range(4):
        idx = mask[row].nonzero().view(-1).tolist()
        running, next_value = 0.0, 0.0
        for i in reversed(idx):
            delta = float(rewards[row, i]) + gamma * next_value - float(values[row, i])
            running = delta + gamma * lam * running
            next_value = float(values[row, i])
            assert abs(float(adv[row, i]) - running) < 1e-5
            assert abs(float(ret[row, i]) - (running + float(values[row, i]))) < 1e-5
    assert float(adv[~mask].abs().max()) == 0.0 and float(ret[~mask].abs().max()) == 0.0
    # garbage at masked positions changes nothing
    noisy_r, noisy_v = rewards.clone(), values.clone()
    noisy_r[~mask], noisy_v[~mask] = 1e6, -1e6
    again, _ = gae_advantages(noisy_r, noisy_v, mask, gamma=gamma, lam=lam)
    assert torch.equal(again, adv)
    # lam = 1, gamma = 1: advantage = reward-to-go minus value
    mc, _ = gae_advantages(rewards, values, mask, gamma=1.0, lam=1.0)
    togo = torch.where(mask, rewards, torch.zeros_like(rewards)).flip(1).cumsum(1).flip(1)
    assert torch.allclose(mc[mask], (togo - values)[mask], atol=1e-5)


def test_kl_shaped_rewards_put_the_sequence_reward_on_the_last_real_token():
    gen, mask = _inputs(1)
    lp, ref = torch.randn(4, 7, generator=gen), torch.randn(4, 7, generator=gen)
    seq = torch.tensor([1.0, -2.0, 0.5, 3.0])
    out = kl_shaped_rewards(seq, lp, ref, mask, kl_coef=0.1)
    last = [6, 3, 6, 6]
    for row in range(4):
        for i in range(7):
            want = 0.0 if not mask[row, i] else -0.1 * float(lp[row, i] - ref[row, i]) + (float(seq[row]) if i == last[row] else 0.0)
            assert abs(float(out[row, i]) - want) < 1e-6
    empty = torch.zeros(1, 3, dtype=torch.bool)
    assert float(kl_shaped_rewards(torch.tensor([5.0]), torch.zeros(1, 3), torch.zeros(1, 3), empty).abs().sum()) == 0.0


def test_whiten_and_value_loss():
    gen, mask = _inputs(2)
    x = torch.randn(4, 7, generator=gen) * 3 + 2
    w = whiten(x, mask)
    assert abs(float(w[mask].mean())) < 1e-5 and abs(float(w[mask].var(unbiased=False)) - 1.0) < 1e-4
    assert float(w[~mask].abs().max()) == 0.0
    keep_mean = whiten(x, mask, shift_mean=False)
    assert abs(float(keep_mean[mask].mean()) - float(x[mask].mean())) < 1e-4
    v, old, ret = torch.randn(4, 7, generator=gen), torch.randn(4, 7, generator=gen), torch.randn(4, 7, generator=gen)
    plain = value_loss(v, old, ret, mask, clip_range=None)
    assert abs(float(plain) - 0.5 * float(((v - ret) ** 2)[mask].mean())) < 1e-6
    clipped = value_loss(v, old, ret, mask, clip_range=0.2)
    vc = old + (v - old).clamp(-0.2, 0.2)
    assert abs(float(clipped) - 0.5 * float(torch.maximum((v - ret) ** 2, (vc - ret) ** 2)[mask].mean())) < 1e-6
    assert float(clipped) >= float(plain)


def test_one_ppo_step_through_the_registry_operator_improves_the_surrogate():
    from rl_engine.kernels.registry import kernel_registry

    gen, mask = _inputs(3)
    logits = torch.randn(4, 7, 11, generator=gen).requires_grad_(True)
    actions = torch.randint(0, 11, (4, 7), generator=gen)
    old = torch.log_softmax(logits.detach(), -1).gather(-1, actions[..., None]).squeeze(-1)
    values = torch.zeros(4, 7)
    rewards = kl_shaped_rewards(torch.tensor([1.0, -1.0, 0.5, -0.5]), old, old, mask, kl_coef=0.0)
    adv, _ = gae_advantages(rewards, values, mask, gamma=1.0, lam=1.0)
    adv = whiten(adv, mask)
    ppo = kernel_registry.get_op("ppo_loss")
    losses = []
    opt = torch.optim.SGD([logits], lr=1.0)
    for _ in range(5):
        lp = torch.log_softmax(logits, -1).gather(-1, actions[..., None]).squeeze(-1)
        loss = ppo(lp, old, adv, mask, clip_eps=0.2)[0]
        losses.append(float(loss.detach()))
        opt.zero_grad()
        loss.backward()
        opt.step()
    assert losses[-1] < losses[0]
