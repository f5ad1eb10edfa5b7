"""Policy-gradient reinforcement learning on small vectorised environments: REINFORCE with a value baseline, advantage
actor-critic, and PPO (clipped surrogate, generalised advantage estimation, several epochs over each batch).
Environments step a whole batch of independent episodes as tensors, so rollouts are one loop over time, not over
episodes. ``CartPole`` integrates the classic cart-and-pole equations (Euler, 0.02 s); ``Corridor`` is a 1-D walk to a goal.
Reference counterpart: scirust-rl-algo/src/lib.rs (``ReinforceAgent``, ``ActorCriticAgent``, ``FeedForwardNet``) and
scirust-learning/src/rl (PPO)."""
from __future__ import annotations

import math

import torch


class Corridor:
    """Positions 0..n-1, start in the middle, actions {left, right}; +1 on reaching the right end, -0.01 per step."""
    obs_dim, n_actions = 1, 2

    def __init__(self, n: int = 7, horizon: int = 40):
        self.n, self.horizon = n, horizon

    def reset(self, batch, generator=None):
        self.pos = torch.full((batch,), self.n // 2, dtype=torch.long)
        self.t = 0
        return self._obs()

    def _obs(self):
        return (self.pos.float() / (self.n - 1))[:, None]

    def step(self, action):
        self.pos = (self.pos + action * 2 - 1).clamp(0, self.n - 1)
        self.t += 1
        goal = self.pos == self.n - 1
        return self._obs(), torch.where(goal, 1.0, -0.01), goal | (self.t >= self.horizon)


class CartPole:
    obs_dim, n_actions = 4, 2

    def __init__(self, horizon: int = 200):
        self.horizon = horizon

    def reset(self, batch, generator=None):
        self.s = (torch.rand(batch, 4, generator=generator) - 0.5) * 0.1
        self.t = 0
        return self.s.clone()

    def step(self, action):
        g, mc, mp, l, f, tau = 9.8, 1.0, 0.1, 0.5, 10.0, 0.02
        x, xd, th, thd = self.s.unbind(1)
        force = (action.float() * 2 - 1) * f
        ct, st = th.cos(), th.sin()
        tmp = (force + mp * l * thd * thd * st) / (mc + mp)
        tha = (g * st - ct * tmp) / (l * (4.0 / 3.0 - mp * ct * ct / (mc + mp)))
        xa = tmp - mp * l * tha * ct / (mc + mp)
        self.s = torch.stack([x + tau * xd, xd + tau * xa, th + tau * thd, thd + tau * tha], 1)
        self.t += 1
        fail = (self.s[:, 0].abs() > 2.4) | (self.s[:, 2].abs() > 12 * math.pi / 180)
        return self.s.clone(), torch.ones(action.shape[0]), fail | (self.t >= self.horizon)


def _mlp(i, h, o):
    return torch.nn.Sequential(torch.nn.Linear(i, h), torch.nn.Tanh(), torch.nn.Linear(h, h), torch.nn.Tanh(), torch.nn.Linear(h, o))


def rollout(env, policy, value, batch, generator=None):
    """-> dict of [T, B] tensors; after an episode ends its later steps carry mask 0."""
    obs = env.reset(batch, generator)
    alive = torch.ones(batch, dtype=torch.bool)
    keys = {k: [] for k in ("obs", "act", "logp", "rew", "val", "mask")}
    while bool(alive.any()):
        with torch.no_grad():
            dist = torch.distributions.Categorical(logits=policy(obs))
            act = dist.sample() if generator is None else torch.multinomial(dist.probs, 1, generator=generator)[:, 0]
            val = value(obs)[:, 0] if value is not None else torch.zeros(batch)
        nxt, rew, done = env.step(act)
        for k, v in zip(keys, (obs, act, dist.log_prob(act), rew, val, alive.float())):
            keys[k].append(v)
        alive = alive & ~done
        obs = nxt
    return {k: torch.stack(v) for k, v in keys.items()}


def discounted_returns(rew, mask, gamma):
    out, run = torch.zeros_like(rew), torch.zeros(rew.shape[1])
    for t in reversed(range(rew.shape[0])):
        run = rew[t] * mask[t] + gamma * run * mask[t]
        out[t] = run
    return out


def gae(rew, val, mask, gamma, lam):
    adv, run = torch.zeros_like(rew), torch.zeros(rew.shape[1])
    nxt = torch.cat([val[1:] * mask[1:], torch.zeros(1, rew.shape[1])])
    for t in reversed(range(rew.shape[0])):
        delta = rew[t] + gamma * nxt[t] - val[t]
        run = (delta + gamma * lam * run) * mask[t]
        adv[t] = run
    return adv, adv + val


class PolicyGradientAgent:
    """``algo``: ``reinforce`` (Monte-Carlo returns minus the value baseline), ``a2c`` (GAE advantages, one step per batch),
    ``ppo`` (GAE, clipped ratio, ``epochs`` passes)."""

    def __init__(self, env, algo: str = "ppo", hidden: int = 32, lr: float = 3e-3, gamma: float = 0.99, lam: float = 0.95,
                 clip: float = 0.2, epochs: int = 4, entropy: float = 0.01, seed: int = 0):
        if algo not in ("reinforce", "a2c", "ppo"):
            raise ValueError(f"unknown algorithm {algo!r}")
        torch.manual_seed(seed)
        self.env, self.algo, self.gamma, self.lam, self.clip, self.epochs, self.entropy = env, algo, gamma, lam, clip, epochs, entropy
        self.policy, self.value = _mlp(env.obs_dim, hidden, env.n_actions), _mlp(env.obs_dim, hidden, 1)
        self.opt = torch.optim.Adam(list(self.policy.parameters()) + list(self.value.parameters()), lr=lr)
        self.gen = torch.Generator().manual_seed(seed)

    def act(self, obs, greedy: bool = True):
        logits = self.policy(torch.as_tensor(obs, dtype=torch.float32).reshape(-1, self.env.obs_dim))
        return logits.argmax(1) if greedy else torch.multinomial(logits.softmax(1), 1, generator=self.gen)[:, 0]

    def train_iteration(self, batch: int = 32) -> float:
        """One batch of episodes and its updates -> mean undiscounted episode return of that batch."""
        ro = rollout(self.env, self.policy, self.value, batch, self.gen)
        mask = ro["mask"]
        if self.algo == "reinforce":
            ret = discounted_returns(ro["rew"], mask, self.gamma)
            adv = ret - ro["val"]
        else:
            adv, ret = gae(ro["rew"], ro["val"], mask, self.gamma, self.lam)
        m = mask.bool()
        obs, act, old_lp = ro["obs"][m], ro["act"][m], ro["logp"][m]
        adv_f, ret_f = adv[m], ret[m]
        adv_f = (adv_f - adv_f.mean()) / adv_f.std().clamp_min(1e-8)
        for _ in range(self.epochs if self.algo == "ppo" else 1):
            dist = torch.distributions.Categorical(logits=self.policy(obs))
            lp = dist.log_prob(act)
            if self.algo == "ppo":
                ratio = torch.exp(lp - old_lp)
                pl = -torch.min(ratio * adv_f, ratio.clamp(1 - self.clip, 1 + self.clip) * adv_f).mean()
            else:
                pl = -(lp * adv_f).mean()
            vl = ((self.value(obs)[:, 0] - ret_f) ** 2).mean()
            loss = pl + 0.5 * vl - self.entropy * dist.entropy().mean()
            self.opt.zero_grad()
            loss.backward()
            torch.nn.utils.clip_grad_norm_(list(self.policy.parameters()) + list(self.value.parameters()), 1.0)
            self.opt.step()
        return float((ro["rew"] * mask).sum(0).mean())

    def train(self, iterations: int, batch: int = 32):
        return [self.train_iteration(batch) for _ in range(iterations)]

    @torch.no_grad()
    def evaluate(self, episodes: int = 16) -> float:
        obs = self.env.reset(episodes, self.gen)
        alive, total = torch.ones(episodes, dtype=torch.bool), torch.zeros(episodes)
        while bool(alive.any()):
            obs, rew, done = self.env.step(self.act(obs))
            total += rew * alive
            alive &= ~done
        return float(total.mean())
