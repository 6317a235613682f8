"""Reinforcement-learning agents: tabular DQN, linear PPO, entropy-jittered SAC and the policy-
gradient learner whose update can run on a hypergradient tape.

Restated from crates/st-spiral-rl/src/algorithms.rs (``DqnAgent`` :31-300, ``PpoAgent`` :306-402,
``SacAgent`` :405-480) and crates/st-spiral-rl/src/lib.rs:150-500 (``SpiralPolicyGradient``:
REINFORCE with the mean return as baseline; deterministic ``cos`` initialisation; optional
``AmegaHypergrad`` tape for the weight update).  Tensors are ``torch`` tensors on any device; the
batched updates are vectorised.
"""
from __future__ import annotations

import math
import zlib
from dataclasses import dataclass
from typing import Optional, Sequence

import torch

from .optim.amegagrad import AmegaHypergrad


class SpiralRlError(ValueError):
    pass


def _rng(label: str) -> torch.Generator:
    return torch.Generator().manual_seed(zlib.crc32(label.encode()))


@dataclass
class EpsilonGreedySchedule:
    start: float = 1.0
    end: float = 0.05
    decay_steps: int = 1000

    def value(self, step: int) -> float:
        t = min(max(step, 0), self.decay_steps) / max(1, self.decay_steps)
        return self.start + (self.end - self.start) * t


@dataclass
class DqnActionTrace:
    state: int
    action: int
    greedy_action: int
    explored: bool
    epsilon: float
    q_values: list


class DqnAgent:
    def __init__(self, state_dim: int, action_dim: int, discount: float, learning_rate: float):
        if state_dim <= 0 or action_dim <= 0:
            raise SpiralRlError(f"invalid state/action shape ({state_dim}, {action_dim})")
        if not 0.0 <= discount <= 1.0:
            raise SpiralRlError(f"discount {discount} is outside [0, 1]")
        if learning_rate <= 0:
            raise SpiralRlError(f"learning rate must be positive, got {learning_rate}")
        self.state_dim, self.action_dim = state_dim, action_dim
        self.discount, self.learning_rate = discount, learning_rate
        self.epsilon = 0.1
        self._schedule: Optional[EpsilonGreedySchedule] = None
        self._schedule_step = 0
        self._table = torch.zeros(state_dim, action_dim)
        self._gen = _rng(f"st-spiral-rl/dqn:{state_dim}:{action_dim}")

    def set_epsilon(self, epsilon: float) -> None:
        self.epsilon = min(max(epsilon, 0.0), 1.0)

    def configure_epsilon_schedule(self, schedule: EpsilonGreedySchedule) -> None:
        self._schedule, self._schedule_step = schedule, 0
        self.epsilon = schedule.value(0)

    def epsilon_schedule(self) -> Optional[EpsilonGreedySchedule]:
        return self._schedule

    def schedule_step(self) -> Optional[int]:
        return self._schedule_step if self._schedule else None

    def _check_state(self, state: int) -> None:
        if not 0 <= state < self.state_dim:
            raise SpiralRlError(f"state {state} is outside [0, {self.state_dim})")

    def q_values(self, state: int) -> list:
        self._check_state(state)
        return self._table[state].tolist()

    def greedy_action(self, state: int) -> int:
        self._check_state(state)
        return int(torch.argmax(self._table[state]))

    def select_action_trace(self, state: int) -> DqnActionTrace:
        greedy = self.greedy_action(state)
        eps = self.epsilon
        explored = float(torch.rand((), generator=self._gen)) < eps
        action = int(torch.randint(0, self.action_dim, (), generator=self._gen)) if explored else greedy
        if self._schedule is not None:
            self._schedule_step += 1
            self.epsilon = self._schedule.value(self._schedule_step)
        return DqnActionTrace(state, action, greedy, explored, eps, self._table[state].tolist())

    def select_action(self, state: int) -> int:
        return self.select_action_trace(state).action

    def select_actions(self, states: Sequence[int]) -> list:
        return [self.select_action(s) for s in states]

    def update(self, state: int, action: int, reward: float, next_state: int) -> None:
        target = reward + self.discount * float(self._table[next_state].max())
        cur = float(self._table[state, action])
        self._table[state, action] = cur + self.learning_rate * (target - cur)

    def update_batch(self, states, actions, rewards, next_states, dones=None) -> None:
        n = len(states)
        if not (len(actions) == len(rewards) == len(next_states) == n) or (dones is not None and len(dones) != n):
            raise SpiralRlError("update_batch: all sequences must have the same length")
        for i in range(n):      # sequential on purpose: later transitions see earlier updates
            nxt = 0.0 if (dones is not None and dones[i]) else float(self._table[next_states[i]].max())
            cur = float(self._table[states[i], actions[i]])
            self._table[states[i], actions[i]] = cur + self.learning_rate * (rewards[i] + self.discount * nxt - cur)

    def table(self) -> torch.Tensor:
        return self._table

    def set_table(self, values) -> None:
        t = torch.as_tensor(values, dtype=torch.float32).reshape(-1)
        if t.numel() != self.state_dim * self.action_dim:
            raise SpiralRlError(f"table needs {self.state_dim * self.action_dim} values, got {t.numel()}")
        self._table = t.reshape(self.state_dim, self.action_dim).clone()


class PpoAgent:
    def __init__(self, state_dim: int, action_dim: int, learning_rate: float, clip_range: float):
        if state_dim <= 0 or action_dim <= 0:
            raise SpiralRlError(f"invalid state/action shape ({state_dim}, {action_dim})")
        g = _rng(f"st-spiral-rl/ppo:init:{state_dim}:{action_dim}")
        self.policy_weights = (torch.rand(action_dim, state_dim, generator=g) - 0.5) * 0.1
        self.value_weights = torch.zeros(state_dim)
        self.state_dim, self.action_dim = state_dim, action_dim
        self.learning_rate, self.clip_range = learning_rate, min(max(clip_range, 0.0), 1.0)

    def score_actions(self, state) -> list:
        return (self.policy_weights @ torch.as_tensor(state, dtype=torch.float32)).tolist()

    def value(self, state) -> float:
        return float(self.value_weights @ torch.as_tensor(state, dtype=torch.float32))

    def log_prob(self, state, action: int) -> float:
        logits = self.policy_weights @ torch.as_tensor(state, dtype=torch.float32)
        return float(logits[action] - torch.logsumexp(logits, 0))

    def update(self, state, action: int, advantage: float, old_log_prob: float) -> None:
        s = torch.as_tensor(state, dtype=torch.float32)
        ratio = math.exp(self.log_prob(s, action) - old_log_prob)
        clipped = min(max(ratio, 1.0 - self.clip_range), 1.0 + self.clip_range)
        self.policy_weights[action] += self.learning_rate * clipped * advantage * s
        self.value_weights += self.learning_rate * advantage * s


class SacAgent:
    def __init__(self, state_dim: int, action_dim: int, temperature: float):
        if temperature <= 0:
            raise SpiralRlError(f"temperature must be positive, got {temperature}")
        self._gen = _rng(f"st-spiral-rl/sac:init:{state_dim}:{action_dim}")
        self.policy_weights = (torch.rand(action_dim, state_dim, generator=self._gen) * 2 - 1) * temperature
        self.state_dim, self.action_dim, self.temperature = state_dim, action_dim, temperature

    def sample_action(self, state) -> int:
        scores = torch.exp(self.policy_weights @ torch.as_tensor(state, dtype=torch.float32) / self.temperature)
        total = float(scores.sum())
        if total <= 1.1920929e-07:
            return 0
        draw = float(torch.rand((), generator=self._gen)) * total
        idx = int(torch.searchsorted(torch.cumsum(scores, 0), torch.tensor(draw)))
        return min(idx, self.action_dim - 1)

    def jitter(self, entropy_target: float) -> None:
        noise = (torch.rand(self.policy_weights.shape, generator=self._gen) * 2 - 1) * self.temperature
        self.policy_weights = torch.tanh(self.policy_weights + noise * entropy_target)


@dataclass
class EpisodeReport:
    total_reward: float
    mean_return: float
    steps: int
    hypergrad_applied: bool
    hyper_surprise: Optional[dict] = None


@dataclass
class PolicyTelemetry:
    state_dim: int
    action_dim: int
    pending_steps: int
    hypergrad: bool
    weight_norm: float


class SpiralPolicyGradient:
    """Linear-softmax REINFORCE.  ``weights`` is ``(state_dim, action_dim)``; episodes are recorded
    with :meth:`record_transition` and applied by :meth:`finish_episode`."""

    def __init__(self, state_dim: int, action_dim: int, learning_rate: float, discount: float, device="cpu"):
        if state_dim <= 0 or action_dim <= 0:
            raise SpiralRlError(f"invalid dimensions ({state_dim}, {action_dim})")
        if learning_rate <= 0:
            raise SpiralRlError(f"learning rate must be positive, got {learning_rate}")
        if not 0.0 <= discount <= 1.0:
            raise SpiralRlError(f"discount {discount} is outside [0, 1]")
        r = torch.arange(1, state_dim + 1, dtype=torch.float32)[:, None]
        c = torch.arange(1, action_dim + 1, dtype=torch.float32)[None, :]
        self.weights = (torch.cos(r * c) * 0.01).clamp(-0.05, 0.05).to(device)
        self.bias = torch.zeros(action_dim, device=device)
        self.state_dim, self.action_dim = state_dim, action_dim
        self.learning_rate, self.discount = learning_rate, discount
        self._episode: list = []
        self._tape: Optional[AmegaHypergrad] = None
        self._surprise_std: Optional[float] = None

    def enable_hypergrad(self, curvature: float, learning_rate: float) -> None:
        self._tape = AmegaHypergrad(curvature, learning_rate, self.state_dim, self.action_dim)

    def attach_hyper_surprise(self, std_threshold: float) -> None:
        """When the standard deviation of an episode's returns exceeds ``std_threshold`` the step is
        damped by ``threshold / std`` (a loss-spread trigger)."""
        self._surprise_std = float(std_threshold)

    def detach_hyper_surprise(self) -> Optional[float]:
        s, self._surprise_std = self._surprise_std, None
        return s

    def reset_episode(self) -> None:
        self._episode.clear()

    def _state_vec(self, state) -> torch.Tensor:
        t = getattr(state, "_t", state)
        t = torch.as_tensor(t, dtype=torch.float32).reshape(-1).to(self.weights.device)
        if t.numel() != self.state_dim:
            raise SpiralRlError(f"state has {t.numel()} features, expected {self.state_dim}")
        return t

    def policy(self, state) -> list:
        return torch.softmax(self._state_vec(state) @ self.weights + self.bias, 0).tolist()

    def select_action(self, state) -> int:
        return int(torch.argmax(self._state_vec(state) @ self.weights + self.bias))

    def record_transition(self, state, action: int, reward: float) -> None:
        if not 0 <= action < self.action_dim:
            raise SpiralRlError(f"action {action} is outside [0, {self.action_dim})")
        s = self._state_vec(state)
        self._episode.append((s, action, float(reward), torch.softmax(s @ self.weights + self.bias, 0)))

    def telemetry(self) -> PolicyTelemetry:
        return PolicyTelemetry(self.state_dim, self.action_dim, len(self._episode), self._tape is not None,
                               float(self.weights.norm()))

    def finish_episode(self, learning_rate: Optional[float] = None) -> EpisodeReport:
        if not self._episode:
            raise SpiralRlError("cannot finish an empty episode")
        lr = self.learning_rate if learning_rate is None else learning_rate
        if not (math.isfinite(lr) and lr > 0):
            raise SpiralRlError(f"learning rate must be positive, got {lr}")
        rewards = torch.tensor([e[2] for e in self._episode], device=self.weights.device)
        returns = torch.empty_like(rewards)
        run = 0.0
        for i in range(len(rewards) - 1, -1, -1):
            run = float(rewards[i]) + self.discount * run
            returns[i] = run
        baseline = float(returns.mean())
        signal = None
        if self._surprise_std is not None and len(returns) > 1:
            std = float(returns.std(unbiased=False))
            if std > self._surprise_std:
                signal = {"std": std, "threshold": self._surprise_std, "scale": self._surprise_std / std}
                lr *= signal["scale"]
        states = torch.stack([e[0] for e in self._episode])                       # [T, S]
        probs = torch.stack([e[3] for e in self._episode])                        # [T, A]
        onehot = torch.nn.functional.one_hot(torch.tensor([e[1] for e in self._episode], device=states.device),
                                             self.action_dim).float()
        coeff = (onehot - probs) * (returns - baseline)[:, None] * lr              # [T, A]
        self.bias += coeff.sum(0)
        wgrad = states.t() @ coeff
        if self._tape is not None:
            self._tape.accumulate_wave(wgrad)
            self._tape.apply(self.weights)
        else:
            self.weights += wgrad
        rep = EpisodeReport(float(rewards.sum()), baseline, len(self._episode), self._tape is not None, signal)
        self._episode.clear()
        return rep
