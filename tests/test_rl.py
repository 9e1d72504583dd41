"""The asynchronous RL stack: metric records, routing, the work buffer, sample packing, environments, the
continuous-batching engine and the controller end to end (all on CPU)."""

import asyncio
import json
import math

import pytest
import torch

from torchtitan_b200.experiments.rl import metrics as m


def run(coro):
    return asyncio.run(coro)


# ---------------------------------------------------------------------------------------------------------- metrics
def test_metric_kinds_merge_observations_not_means():
    recs = [m.Metric("r", m.Mean.from_list([1, 1, 1])), m.Metric("r", m.Mean(2.0)), m.Metric("r", m.Mean(6.0, count=2)),
            m.Metric("r", m.Max.from_list([1.0, 4.0])), m.Metric("r", m.Max.from_list([])), m.Metric("r", m.Min(0.5)),
            m.Metric("n", m.Sum(2)), m.Metric("n", m.Sum.from_list([1, 1])),
            m.Metric("s", m.Std.from_list([1.0, 2.0])), m.Metric("s", m.Std(7.0, count=2, sum_squares=25.0)),
            m.Metric("a", m.SummaryStats.from_list([1.0, 3.0])), m.Metric("a", m.SummaryStats(5.0)),
            m.Metric("loss", m.NoReduce(0.25))]
    out = m.aggregate(recs)
    assert out["r/mean"] == pytest.approx((3 + 2 + 6) / 6) and out["r/max"] == 4.0 and out["r/min"] == 0.5
    assert out["n/sum"] == 4.0 and out["loss"] == 0.25
    assert out["s/std"] == pytest.approx(torch.tensor([1.0, 2.0, 3.0, 4.0]).std(unbiased=False).item())
    assert out["a/_mean"] == 3.0 and out["a/_max"] == 5.0 and out["a/_min"] == 1.0 and out["a/_sum"] == 9.0
    assert math.isnan(m.aggregate([m.Metric("e", m.Mean.from_list([]))])["e/mean"])
    assert m.aggregate([m.Metric("e", m.SummaryStats.from_list([]))])["e/_sum"] == 0.0
    with pytest.raises(ValueError):
        m.aggregate([m.Metric("loss", m.NoReduce(1)), m.Metric("loss", m.NoReduce(2))])
    with pytest.raises(ValueError):
        m.Std(1.0, count=2)


def test_metrics_processor_writes_jsonl_and_prefixes_validation(tmp_path):
    p = m.MetricsProcessor(dump_folder=str(tmp_path))
    p.log(step=1, metrics=[m.Metric("loss/mean", m.NoReduce(0.5)), m.Metric("x", m.Mean.from_list([]))])
    flat = p.log(step=1, metrics=[m.Metric("rollout_reward", m.SummaryStats.from_list([1, 0]))], is_validation=True)
    assert flat["validation/rollout_reward/_mean"] == 0.5
    rows = [json.loads(ln) for ln in open(tmp_path / "rl_metrics.jsonl")]
    assert rows[0]["loss/mean"] == 0.5 and rows[0]["x/mean"] is None and rows[1]["validation"] is True
    t = m.MetricsTimer()
    with t.record("timing/a"):
        pass
    assert [x.key for x in t.flush()] == ["timing/a"] and t.flush() == []


# ---------------------------------------------------------------------------------------------------------- routing
class _Cand:
    def __init__(self, load=0):
        self.reserved_load = load


def test_routing_strategies():
    from torchtitan_b200.experiments.rl import (LeastLoadedRoutingStrategy, RoundRobinRoutingStrategy, RoutingContext,
                                                StickySessionRoutingStrategy)

    a, b, c = _Cand(), _Cand(), _Cand()
    rr = RoundRobinRoutingStrategy()
    assert [rr.choose(RoutingContext(), [a, b, c]) for _ in range(4)] == [a, b, c, a]
    ll = LeastLoadedRoutingStrategy()
    # all idle: ties rotate by recency instead of always returning the first candidate
    assert [ll.choose(RoutingContext(), [a, b, c]) for _ in range(4)] == [a, b, c, a]
    b.reserved_load = 2
    assert ll.choose(RoutingContext(), [a, b, c]) in (a, c) and ll.choose(RoutingContext(), [b]) is b
    st = StickySessionRoutingStrategy(StickySessionRoutingStrategy.Config(max_sessions=2))
    first = st.choose(RoutingContext(session_id="s1"), [a, b, c])
    first.reserved_load += 5
    assert st.choose(RoutingContext(session_id="s1"), [a, b, c]) is first          # pinned although loaded
    rest = [x for x in (a, b, c) if x is not first]
    moved = st.choose(RoutingContext(session_id="s1"), rest)                       # its replica left the rotation
    assert moved in rest and st.choose(RoutingContext(session_id="s1"), [a, b, c]) is moved
    st.choose(RoutingContext(session_id="s2"), [a, b, c])
    st.choose(RoutingContext(session_id="s3"), [a, b, c])                          # evicts s1 (least recently used)
    assert "s1" not in st._sessions and len(st._sessions) == 2
    with pytest.raises(ValueError):
        StickySessionRoutingStrategy.Config(max_sessions=0)


def test_intra_generator_router_tracks_reservations():
    from torchtitan_b200.experiments.rl import IntraGeneratorRouter, LeastLoadedRoutingStrategy

    r = IntraGeneratorRouter(IntraGeneratorRouter.Config(strategy=LeastLoadedRoutingStrategy.Config()), dp_degree=2)
    ranks = [r.reserve(f"q{i}") for i in range(4)]
    assert sorted(ranks) == [0, 0, 1, 1] and r.loads() == [2, 2]
    r.release("q0")
    assert r.reserve("q4") == ranks[0]
    with pytest.raises(ValueError):
        r.reserve("q4")
    sticky = IntraGeneratorRouter(dp_degree=3)
    assert len({sticky.reserve(f"t{i}", routing_session_id="same") for i in range(5)}) == 1
    with pytest.raises(ValueError):
        IntraGeneratorRouter(dp_degree=1)


class _FakeGen:
    def __init__(self, name, delay=0.01, fail=False):
        self.name, self.delay, self.fail = name, delay, fail
        self.calls, self.version, self.pulled_while_busy = 0, 0, False
        self.inflight = 0

    async def generate(self, prompt, *, request_id, routing_session_id=None, sampling_config=None):
        from torchtitan_b200.experiments.rl import Completion

        self.calls += 1
        self.inflight += 1
        try:
            await asyncio.sleep(self.delay)
            if self.fail:
                raise RuntimeError("boom")
            return Completion(request_id=request_id, token_ids=[1], token_logprobs=[0.0], finish_reason="stop",
                              min_policy_version=self.version, max_policy_version=self.version)
        finally:
            self.inflight -= 1

    async def pull_model_state_dict(self, version):
        self.pulled_while_busy |= self.inflight > 0
        await asyncio.sleep(0.005)
        self.version = version

    async def close(self):
        return self.name


def test_inter_generator_router_balances_releases_on_failure_and_drains():
    from torchtitan_b200.experiments.rl import InterGeneratorRouter

    async def go():
        g0, g1 = _FakeGen("a"), _FakeGen("b")
        router = InterGeneratorRouter(generators=[g0, g1])
        await asyncio.gather(*(router.generate([1], request_id=f"r{i}") for i in range(6)))
        assert (g0.calls, g1.calls) == (3, 3) and router.loads() == [0, 0]
        bad = InterGeneratorRouter(generators=[_FakeGen("x", fail=True)])
        with pytest.raises(RuntimeError):
            await bad.generate([1], request_id="q")
        assert bad.loads() == [0]                                     # the failed call left no load behind
        # without hot swap a replica is drained before its pull, and requests keep being served meanwhile
        slow, fast = _FakeGen("slow", delay=0.05), _FakeGen("fast", delay=0.001)
        cold = InterGeneratorRouter(InterGeneratorRouter.Config(hot_swap=False), generators=[slow, fast])
        busy = [asyncio.create_task(cold.generate([1], request_id=f"b{i}")) for i in range(2)]
        await asyncio.sleep(0.005)
        pull = asyncio.create_task(cold.pull_model_state_dict(7))
        await asyncio.sleep(0.01)
        late = await cold.generate([1], request_id="late")
        await asyncio.gather(pull, *busy)
        assert not slow.pulled_while_busy and not fast.pulled_while_busy
        assert slow.version == fast.version == 7 and late is not None
        hot = InterGeneratorRouter(generators=[_FakeGen("h", delay=0.05)])
        t = asyncio.create_task(hot.generate([1], request_id="h0"))
        await asyncio.sleep(0.005)
        await hot.pull_model_state_dict(3)
        await t
        assert hot._replicas[0].generator.pulled_while_busy            # hot swap does not wait
        assert await router.close_generators() == ["a", "b"]

    run(go())


# ------------------------------------------------------------------------------------------------------ work buffer
def test_work_buffer_slots_outlive_entries_and_window_is_anchored():
    from torchtitan_b200.experiments.rl import RolloutGroup, RolloutGroupWork, RolloutGroupWorkBuffer

    async def go():
        buf = RolloutGroupWorkBuffer(max_active_rollout_groups=4, window_size=2)
        for g in range(4):
            assert await buf.wait_for_slot()
            await buf.add_work(RolloutGroupWork(group_id=g, sample=g))
        with pytest.raises(RuntimeError):
            await buf.add_work(RolloutGroupWork(group_id=9, sample=9))
        claimed = [await buf.claim_next() for _ in range(4)]
        assert [w.group_id for w in claimed] == [0, 1, 2, 3]
        # groups 1 and 3 finish first: 1 is inside the window [0, 1], 3 is not
        await buf.finalize_work(RolloutGroup(group_id=3, rollouts=[]))
        await buf.finalize_work(RolloutGroup(group_id=1, rollouts=[]))
        assert (await buf.take_finalized()).group_id == 1
        blocked = asyncio.create_task(buf.take_finalized())
        await asyncio.sleep(0.01)
        assert not blocked.done()                                   # the window stays anchored at the unfinished head 0
        await buf.finalize_work(RolloutGroup(group_id=0, rollouts=[]))
        assert (await blocked).group_id == 0
        # taking entries did not free slots
        waiter = asyncio.create_task(buf.wait_for_slot())
        await asyncio.sleep(0.01)
        assert not waiter.done()
        await buf.release_active_groups(2, reason="trained")
        assert await waiter
        flat = m.aggregate(buf.metrics())
        assert flat["rollout_buffer/available_active_slots"] == 2 and flat["rollout_buffer/active_slots_in_use_peak"] == 4
        with pytest.raises(RuntimeError):
            await buf.release_active_groups(5, reason="x")
        stuck = asyncio.create_task(buf.claim_next())
        await asyncio.sleep(0.01)
        await buf.close()
        assert await stuck is None and await buf.take_finalized() is None and not await buf.wait_for_slot()

    run(go())
    with pytest.raises(ValueError):
        RolloutGroupWorkBuffer(max_active_rollout_groups=2, window_size=3)


# ---------------------------------------------------------------------------------------------------------- packing
def _turn(g, r, t, prompt, comp, v=0):
    from torchtitan_b200.experiments.rl import RolloutTurn, RolloutTurnID

    return RolloutTurn(rollout_id=RolloutTurnID(group_id=g, rollout_id=r, turn_id=t), prompt_token_ids=prompt,
                       completion_token_ids=comp, completion_logprobs=[-0.5] * len(comp), min_policy_version=v,
                       max_policy_version=v)


def _rollout(g, r, turns, reward, adv):
    from torchtitan_b200.experiments.rl import Rollout, RolloutStatus

    return Rollout(group_id=g, rollout_id=r, status=RolloutStatus.COMPLETED, turns=turns, reward=reward, advantage=adv)


def test_sample_builder_merges_growing_prefix_and_branches_where_it_breaks():
    from torchtitan_b200.experiments.rl import RolloutGroup, TrainingSampleBuilder

    P1, C1, E1, C2, P2, C4 = [1, 2], [3], [4, 5], [6, 7], [9], [8]
    turns = [_turn(0, 0, 0, P1, C1, v=5), _turn(0, 0, 1, P1 + C1 + E1, C2, v=6), _turn(0, 0, 2, P2, C4, v=7)]
    b = TrainingSampleBuilder()
    s = b.rollout_to_training_samples(_rollout(0, 0, turns, 1.0, 0.5))
    assert len(s) == 2
    assert s[0].token_ids == P1 + C1 + E1 + C2
    assert s[0].loss_mask == [False, False, True, False, False, True, True]
    assert s[0].advantage == [0, 0, 0.5, 0, 0, 0.5, 0.5] and s[0].logprobs[2] == -0.5 and s[0].logprobs[3] == 0.0
    assert (s[0].min_policy_version, s[0].max_policy_version) == (5, 6) and s[0].rollout_id.turn_id == 0
    assert s[1].token_ids == P2 + C4 and s[1].rollout_id.turn_id == 2 and s[1].min_policy_version == 7
    # group filters
    same = RolloutGroup(group_id=1, rollouts=[_rollout(1, i, [_turn(1, i, 0, P1, C1)], 1.0, 0.0) for i in range(2)])
    out = b.build_from_group(rollout_group=same)
    assert out.training_samples == [] and m.aggregate(out.metrics)["training_sample_builder/num_groups_dropped_zero_std/sum"] == 1
    kept = TrainingSampleBuilder(TrainingSampleBuilder.Config(drop_zero_std_reward_groups=False)).build_from_group(rollout_group=same)
    assert len(kept.training_samples) == 2
    blank = RolloutGroup(group_id=2, rollouts=[_rollout(2, 0, [_turn(2, 0, 0, P1, [])], 0.0, 0.0),
                                               _rollout(2, 1, [_turn(2, 1, 0, P1, C1)], 1.0, 0.0)])
    assert b.build_from_group(rollout_group=blank).training_samples == []
    assert b.build_from_group(rollout_group=RolloutGroup(group_id=3, rollouts=[])).training_samples == []
    with pytest.raises(ValueError):
        b.rollout_to_training_samples(_rollout(0, 0, turns, 1.0, None))


def test_batcher_packs_rows_shifts_labels_and_deals_the_grid():
    from torchtitan_b200.experiments.rl import BatchConfig, Batcher, TrainingSample, TrainingSampleGroup
    from torchtitan_b200.experiments.rl.records import RolloutTurnID

    def sample(g, toks, n_prompt, v=0):
        n = len(toks)
        mask = [False] * n_prompt + [True] * (n - n_prompt)
        return TrainingSample(rollout_id=RolloutTurnID(group_id=g, rollout_id=0), min_policy_version=v, max_policy_version=v,
                              token_ids=toks, loss_mask=mask, logprobs=[-1.0 if x else 0.0 for x in mask],
                              advantage=[2.0 if x else 0.0 for x in mask])

    bt = Batcher(Batcher.Config(batch=BatchConfig(local_batch_size=1, seq_len=8)), num_prompts_per_train_step=2,
                 dp_degree=2, pad_id=0)
    g0 = TrainingSampleGroup(0, [sample(0, [10, 11, 12], 1), sample(0, [20, 21, 22], 1, v=1)], [m.Metric("k", m.Sum(1))])
    empty = TrainingSampleGroup(1, [], [m.Metric("k", m.Sum(1))])
    g2 = TrainingSampleGroup(2, [sample(2, list(range(30, 38)), 2), sample(2, list(range(40, 60)), 2)], [])
    assert bt.add_training_samples(training_sample_group=g0) is None
    assert bt.add_training_samples(training_sample_group=empty) is None          # metrics ride along, no sample
    batch = bt.add_training_samples(training_sample_group=g2)                    # the 20-token sample is dropped
    flat = m.aggregate(batch.metrics)
    assert flat["batcher/num_samples_dropped_oversized/sum"] == 1 and flat["k/sum"] == 2
    assert flat["train_batch/num_rollout_groups"] == 2 and flat["train_batch/num_metric_only_groups"] == 1
    assert batch.min_policy_versions == [0, 1, 0]
    # rows: [s0 (2 tokens) + s1 (2)] and [s2 (7)]; one microbatch of two ranks
    assert len(batch.microbatches) == 1 and len(batch.microbatches[0]) == 2
    r0, r1 = batch.microbatches[0]
    assert r0.token_ids.tolist() == [10, 11, 20, 21, 0, 0, 0, 0] and r0.labels.tolist() == [11, 12, 21, 22, 0, 0, 0, 0]
    assert r0.positions.tolist() == [0, 1, 0, 1, 0, 1, 2, 3]
    assert r0.loss_mask.tolist() == [True, True, True, True, False, False, False, False]
    assert r0.advantages[:4].tolist() == [2.0] * 4 and r0.generator_logprobs[:4].tolist() == [-1.0] * 4
    assert r1.token_ids.tolist()[:7] == list(range(30, 37)) and r1.loss_mask.tolist() == [False] + [True] * 6 + [False]
    assert batch.num_global_valid_tokens == 4 + 6
    assert flat["train_batch/padding_frac"] == pytest.approx((16 - 11) / 16)
    # per-sample padding (batch-invariant mode) aligns every sample to the multiple
    pad = Batcher(Batcher.Config(batch=BatchConfig(local_batch_size=1, seq_len=8), per_sample_pad_multiple=4),
                  num_prompts_per_train_step=1, dp_degree=1, pad_id=0)
    b2 = pad.add_training_samples(training_sample_group=g0)
    assert b2.microbatches[0][0].positions.tolist() == [0, 1, 2, 3, 0, 1, 2, 3]
    assert b2.microbatches[0][0].loss_mask.tolist() == [True, True, False, False] * 2


# ----------------------------------------------------------------------------------------------------- environments
class _EchoEnv:
    """Two-turn environment: asks once more after the first answer."""

    def __init__(self, turns=2, slow=False):
        self.turns, self.slow, self.n, self.closed = turns, slow, 0, False

    async def init(self):
        from torchtitan_b200.experiments.rl import MessageEnvInit

        return MessageEnvInit(init_prompt_messages=[{"role": "user", "content": "hi"}])

    async def step(self, message):
        from torchtitan_b200.experiments.rl import MessageEnvStep

        if self.slow:
            await asyncio.sleep(1.0)
        self.n += 1
        if self.n >= self.turns:
            return MessageEnvStep(done=True, env_rewards={"ok": 1.0})
        return MessageEnvStep(env_messages=[{"role": "user", "content": "again"}])

    async def close(self):
        self.closed = True


def _completion(renderer, text, reason="stop"):
    from torchtitan_b200.experiments.rl import Completion

    return Completion(request_id="r", token_ids=renderer._encode(text), token_logprobs=[0.0] * len(text.encode()),
                      finish_reason=reason)


def test_renderer_and_token_env_cover_every_way_an_episode_ends():
    from torchtitan_b200.components.tokenizer import ByteTokenizer
    from torchtitan_b200.experiments.rl import ChatRenderer, MessageEnvStep, RolloutStatus, TokenEnv

    rend = ChatRenderer(tokenizer=ByteTokenizer())
    parsed = rend.parse_response(token_ids=rend._encode(
        '<think>hm</think>fine<tool_call>{"name": "f", "arguments": {"x": 1}}</tool_call><|im_end|>') + [257])
    assert parsed.content == "fine" and parsed.reasoning_content == "hm" and parsed.tool_calls[0]["name"] == "f"
    with pytest.raises(ValueError):
        rend.parse_response(token_ids=rend._encode("<tool_call>{not json}</tool_call>"))
    with pytest.raises(ValueError):
        MessageEnvStep(env_messages=[{"role": "assistant", "content": "x"}])

    async def go():
        env = TokenEnv(message_env=_EchoEnv(), renderer=rend)
        first = await env.init()
        assert first.status is RolloutStatus.ONGOING and first.next_prompt_token_ids[0] == 256
        text = ByteTokenizer().decode(first.next_prompt_token_ids)
        assert text == "<|im_start|>user\nhi<|im_end|>\n<|im_start|>assistant\n"
        c1 = _completion(rend, "one<|im_end|>")
        second = await env.step(c1)
        # token in, token out: the next prompt extends the previous prompt and completion verbatim
        assert second.status is RolloutStatus.ONGOING
        assert second.next_prompt_token_ids[:len(first.next_prompt_token_ids) + len(c1.token_ids)] == \
            first.next_prompt_token_ids + c1.token_ids
        assert ByteTokenizer().decode(second.next_prompt_token_ids).endswith(
            "one<|im_end|>\n<|im_start|>user\nagain<|im_end|>\n<|im_start|>assistant\n")
        last = await env.step(_completion(rend, "two"))
        assert last.status is RolloutStatus.COMPLETED and last.env_rewards == {"ok": 1.0} and last.next_prompt_token_ids is None

        async def end(cfg=None, completion=None, env=None):
            e = TokenEnv(cfg, message_env=env or _EchoEnv(turns=3), renderer=rend)
            out = await e.init()
            if out.status.is_terminal():
                return out.status
            return (await e.step(completion or _completion(rend, "x"))).status

        assert await end(completion=_completion(rend, "cut", reason="length")) is RolloutStatus.TRUNCATED_LENGTH
        assert await end(completion=_completion(rend, "x", reason="abort")) is RolloutStatus.ERROR_ABORT
        assert await end(completion=_completion(rend, "<tool_call>{bad</tool_call>")) is RolloutStatus.ERROR_PARSE
        assert await end(TokenEnv.Config(max_num_turns=1)) is RolloutStatus.TRUNCATED_MAX_TURNS
        assert await end(TokenEnv.Config(max_rollout_tokens=10)) is RolloutStatus.TRUNCATED_PROMPT_TOO_LONG
        assert await end(TokenEnv.Config(max_rollout_tokens=80)) is RolloutStatus.TRUNCATED_PROMPT_TOO_LONG   # second prompt
        assert await end(TokenEnv.Config(step_timeout_s=0.01), env=_EchoEnv(slow=True)) is RolloutStatus.ERROR_TIMEOUT

    run(go())
    assert RolloutStatus.TRUNCATED_MAX_TURNS.is_truncated() and RolloutStatus.ERROR_PARSE.is_error()
    assert not RolloutStatus.ONGOING.is_terminal() and RolloutStatus.COMPLETED.is_terminal()
    # a renderer that drops earlier reasoning cannot bridge: the caller re-renders
    no_think = ChatRenderer(ChatRenderer.Config(preserve_all_thinking=False), tokenizer=ByteTokenizer())
    assert no_think.bridge_to_next_turn(previous_prompt_ids=[1], previous_completion_ids=[2], new_messages=[]) is None


def test_rubric_weights_short_circuits_and_advantages():
    from dataclasses import dataclass

    from torchtitan_b200.experiments.rl import AdvantageEstimator, RewardFn, RolloutGroup, RolloutStatus, Rubric

    class Length(RewardFn):
        @dataclass(kw_only=True, slots=True)
        class Config(RewardFn.Config):
            pass

        async def __call__(self, rollout, env_input):
            return float(len(rollout.turns))

    class Target(RewardFn):
        @dataclass(kw_only=True, slots=True)
        class Config(RewardFn.Config):
            pass

        async def __call__(self, rollout, env_input):
            return float(env_input)

    rubric = Rubric.Config(reward_fns=[Length.Config(weight=3.0), Target.Config(weight=1.0)], truncation_reward=-1.0).build()
    ok = _rollout(0, 0, [_turn(0, 0, 0, [1], [2])], None, None)
    cut = _rollout(0, 1, [], None, None)
    cut.status = RolloutStatus.TRUNCATED_LENGTH
    err = _rollout(0, 2, [], None, None)
    err.status = RolloutStatus.ERROR
    out = run(rubric.score_group([ok, cut, err], 4.0))
    assert out[0].reward == pytest.approx(0.75 * 1 + 0.25 * 4) and out[0].reward_breakdown == {"Length": 1.0, "Target": 4.0}
    assert out[1].reward == -1.0 and out[1].reward_breakdown == {"truncated": -1.0}
    assert out[2].reward == pytest.approx(0.25 * 4)                    # no error_reward configured: the functions run
    with pytest.raises(ValueError):
        Rubric.Config(reward_fns=[]).build()
    with pytest.raises(ValueError):
        Rubric.Config(reward_fns=[Length.Config(), Length.Config()]).build()
    g = RolloutGroup(group_id=0, rollouts=[_rollout(0, i, [], r, None) for i, r in enumerate([1.0, 3.0])])
    assert AdvantageEstimator()(g) == [-1.0, 1.0]
    std = AdvantageEstimator(AdvantageEstimator.Config(should_std_normalize=True))(g)
    assert std[1] == pytest.approx(1.0, abs=1e-5)


# ------------------------------------------------------------------------------------------------------------ engine
def _tiny_llama(seed=0, layers=2):
    from torchtitan_b200.models import get_model_spec

    spec = get_model_spec("llama3", "debugmodel")
    spec.model.layers = spec.model.layers[:layers]
    spec.model.n_layers = layers
    model = spec.model.build()
    model.init_states(seed=seed)
    return spec, model


def test_engine_batches_sequences_and_matches_single_sequence_decoding():
    """Requests of different lengths that arrive together and later decode in shared steps; greedy outputs and
    log-probabilities equal those of the one-sequence cached generator; limits, stop sequences and seeds work."""
    from torchtitan_b200.experiments.rl import CachedGenerator, GenerationEngine, SamplingConfig

    _, model = _tiny_llama()
    prompts = [[5, 9, 11, 4], [7], [3, 3, 8, 1, 2, 6, 6, 10, 12]]
    want = [CachedGenerator(model, temperature=0.0).generate(torch.tensor(p), 6) for p in prompts]
    greedy = SamplingConfig(temperature=0.0, max_tokens=6)

    async def go():
        eng = GenerationEngine(GenerationEngine.Config(max_num_seqs=2, threaded=False), model=model)
        first = [asyncio.create_task(eng.generate(p, request_id=f"r{i}", sampling_config=greedy))
                 for i, p in enumerate(prompts[:2])]
        await asyncio.sleep(0)
        late = asyncio.create_task(eng.generate(prompts[2], request_id="r2", sampling_config=greedy))   # waits for a seat
        got = await asyncio.gather(*first, late)
        for g, w in zip(got, want):
            assert g.token_ids == w.response.tolist() and g.finish_reason == "length"
            assert torch.allclose(torch.tensor(g.token_logprobs), w.logprobs, atol=1e-4)
        assert eng.steps < 18                                         # 3 x 6 tokens in shared steps
        # a stop sequence ends the request after the tokens that complete it
        stop = want[0].response.tolist()[1:3]
        s = await eng.generate(prompts[0], request_id="s", sampling_config=SamplingConfig(temperature=0.0, max_tokens=6,
                                                                                          stop_sequences=[stop]))
        assert s.token_ids == want[0].response.tolist()[:3] and s.finish_reason == "stop"
        # seeded sampling is reproducible, different seeds differ
        a, b, c = await asyncio.gather(*(eng.generate(prompts[0], request_id=f"x{i}", sampling_config=SamplingConfig(
            temperature=1.0, top_k=50, top_p=0.9, max_tokens=12, seed=sd)) for i, sd in enumerate([1, 1, 2])))
        assert a.token_ids == b.token_ids and a.token_ids != c.token_ids and all(lp <= 0 for lp in a.token_logprobs)
        # weights arrive between steps: a request in flight reports both versions
        pulled = []
        eng.weight_source = lambda e: pulled.append(e.policy_version)
        long = asyncio.create_task(eng.generate(prompts[1], request_id="v", sampling_config=SamplingConfig(
            temperature=0.0, max_tokens=8)))
        await asyncio.sleep(0)
        await asyncio.sleep(0)
        await eng.pull_model_state_dict(5)
        done = await long
        assert pulled == [0] and eng.policy_version == 5
        assert done.min_policy_version == 0 and done.max_policy_version == 5
        await eng.close()
        gone = await eng.generate([1], request_id="late")
        assert gone.finish_reason == "abort"

    run(go())


def test_engine_step_failure_fails_the_requests_in_flight_and_the_engine_stays_up():
    from torchtitan_b200.experiments.rl import GenerationEngine, SamplingConfig

    _, model = _tiny_llama()
    greedy = SamplingConfig(temperature=0.0, max_tokens=3)

    async def go():
        for threaded in (False, True):
            eng = GenerationEngine(GenerationEngine.Config(threaded=threaded), model=model)
            with pytest.raises(RuntimeError, match="generation failed"):
                await asyncio.wait_for(eng.generate([5000], request_id="bad", sampling_config=greedy), timeout=20)   # id outside the vocabulary
            ok = await asyncio.wait_for(eng.generate([5, 6], request_id="good", sampling_config=greedy), timeout=20)
            assert len(ok.token_ids) == 3
            await eng.close()

    run(go())


def test_engine_in_a_thread_serves_concurrent_requests():
    from torchtitan_b200.experiments.rl import GenerationEngine, SamplingConfig

    _, model = _tiny_llama()

    async def go():
        eng = GenerationEngine(model=model, eos_id=None)
        out = await asyncio.gather(*(eng.generate([i + 1, 2, 3], request_id=f"t{i}",
                                                  sampling_config=SamplingConfig(temperature=0.0, max_tokens=4)) for i in range(5)))
        assert all(len(c.token_ids) == 4 for c in out)
        flat = m.aggregate([x for c in out for x in c.metrics])
        assert flat["generator/response_length/max"] == 4 and flat["generator/request_latency_s/mean"] > 0
        await eng.close()

    run(go())


# ------------------------------------------------------------------------------------------------------- end to end
def _rl_parts(tmp_path, *, steps, prompts_per_step=2, group=4, drop_flat=False, lr=1e-2):
    from dataclasses import dataclass

    from torchtitan_b200.components.optimizer import OptimizersContainer
    from torchtitan_b200.components.tokenizer import ByteTokenizer
    from torchtitan_b200.config import Configurable
    from torchtitan_b200.experiments.rl import (AsyncController, AsyncLoopConfig, BatchConfig, Batcher, GenerationEngine,
                                                MessageEnv, MessageEnvInit, MessageEnvStep, PolicyLoss, PolicyTrainer,
                                                RewardFn, Rollouter, Rubric, SamplingConfig, TrainingSampleBuilder,
                                                ValidationConfig)
    from torchtitan_b200.parallel.parallel_dims import ParallelDims
    from torchtitan_b200.parallel.parallelize import parallelize_decoder
    from torchtitan_b200.trainer import Trainer

    class Prompts(Configurable):
        @dataclass(kw_only=True, slots=True)
        class Config(Configurable.Config):
            seed: int = 0

        def __init__(self, config, **_):
            self.i = config.seed

        def __next__(self):
            self.i += 1
            return f"q{self.i % 5}"

    class OneShot(MessageEnv):
        @dataclass(kw_only=True, slots=True)
        class Config(MessageEnv.Config):
            pass

        def __init__(self, config=None, *, env_input):
            self.q = env_input

        async def init(self):
            return MessageEnvInit(init_prompt_messages=[{"role": "user", "content": self.q}])

        async def step(self, message):
            return MessageEnvStep(done=True)

    class LowBytes(RewardFn):
        """Share of the completion's tokens from the lower half of the vocabulary: a dense signal that a few steps raise."""

        @dataclass(kw_only=True, slots=True)
        class Config(RewardFn.Config):
            pass

        async def __call__(self, rollout, env_input):
            ids = rollout.turns[-1].completion_token_ids if rollout.turns else []
            return sum(t < 1024 for t in ids) / max(len(ids), 1)

    torch.manual_seed(0)                        # sampling draws from the global generator
    spec, _ = _tiny_llama()
    cfg = Trainer.Config()
    cfg.training.mixed_precision_param = "float32"
    cfg.training.num_tokens_per_microbatch_per_dp_rank = 128
    cfg.training.max_context_length = 128
    pdims = ParallelDims(world_size=1)
    with torch.device("meta"):
        model = spec.model.build()
    eng = parallelize_decoder(model, pdims=pdims, job_config=cfg, device=torch.device("cpu"), seed=3)
    opt = OptimizersContainer(OptimizersContainer.Config(lr=lr, weight_decay=0.0), engines=[eng])
    trainer = PolicyTrainer(model=model, engine=eng, optimizers=opt, loss=PolicyLoss(0.2, 0.28), pdims=pdims)
    generator = GenerationEngine(GenerationEngine.Config(threaded=False), model=model)     # shares the trainer's weights
    config = AsyncController.Config(
        rollouter=Rollouter.Config(train_dataset=Prompts.Config(seed=0), validation_dataset=Prompts.Config(seed=100),
                                   rubric=Rubric.Config(reward_fns=[LowBytes.Config()]), message_env=OneShot.Config()),
        async_loop=AsyncLoopConfig(num_training_steps=steps, num_prompts_per_train_step=prompts_per_step,
                                   num_samples_per_prompt=group, target_offpolicy_steps=1, window_fraction=0.5,
                                   training_sample_builder=TrainingSampleBuilder.Config(drop_zero_std_reward_groups=drop_flat),
                                   max_consecutive_untrainable_groups=16,
                                   batcher=Batcher.Config(batch=BatchConfig(local_batch_size=2, seq_len=64)),
                                   validation=ValidationConfig(num_samples=4)),
        sampling=SamplingConfig(temperature=1.0, max_tokens=6), dump_folder=str(tmp_path), trainer_in_thread=False)
    return AsyncController(config, trainer=trainer, generators=[generator], tokenizer=ByteTokenizer()), trainer, generator


def test_async_controller_trains_with_bounded_staleness(tmp_path):
    ctl, trainer, generator = _rl_parts(tmp_path, steps=10, group=8)
    lc = ctl.config.async_loop
    assert (lc.max_active_rollout_groups, lc.window_size, lc.max_offpolicy_steps) == (4, 2, 2)
    summary = run(ctl.run())
    assert trainer.policy_version == 10 and generator.policy_version == 10
    hist = [h for h in ctl.metrics.history if "loss/mean" in h]
    assert [h["step"] for h in hist] == list(range(1, 11))
    assert all(h["policy_age_max"] <= lc.max_offpolicy_steps for h in hist)
    assert all(math.isfinite(h["loss/mean"]) for h in hist) and any(h["optim/grad_norm"] > 0 for h in hist)
    assert all(0 <= h["train_batch/padding_frac"] < 1 and h["train_batch/num_rollout_groups"] == 2 for h in hist)
    assert "perf/trainer/tokens_per_second_full_step" in hist[0] and "timing/weight_sync/generator_pull" in hist[0]
    # samples generated by the current weights reproduce the generator's log-probabilities exactly in the trainer
    fresh = [h for h in hist if h["policy_age_max"] == 0]
    assert fresh and all(abs(h["bit_wise/logprob_diff/max"]) < 1e-4 and h["loss/ratio_clipped_frac"] == 0 for h in fresh)
    # the policy learned to prefer the rewarded half of the vocabulary
    first = sum(h["rollout_reward/_mean"] for h in hist[:3]) / 3
    last = sum(h["rollout_reward/_mean"] for h in hist[-3:]) / 3
    assert last > first, (first, last)
    assert "validation/rollout_reward/_mean" in summary["pre"] and "validation/rollout_reward/_mean" in summary["post"]
    rows = [json.loads(ln) for ln in open(tmp_path / "rollout_samples.jsonl")]
    assert any(r["is_validation"] for r in rows) and any(not r["is_validation"] for r in rows)
    assert rows[0]["turns"][0]["prompt_messages"][0]["role"] == "user" and "prompt_token_ids" not in rows[0]["turns"][0]
    assert ctl._buffer.released["trained"] == 10 * 2
    run(ctl.close())


def test_async_controller_stops_when_no_group_carries_signal(tmp_path):
    """A constant reward makes every group's rewards equal; with such groups dropped nothing is ever trainable, and the
    job stops with an error instead of generating forever."""
    ctl, trainer, _ = _rl_parts(tmp_path, steps=2, drop_flat=True, lr=0.0)
    ctl.rollouter.rubric.fns[0].__class__.__call__ = lambda self, rollout, env_input: _const()
    with pytest.raises(RuntimeError, match="nothing to train on"):
        run(ctl.run())
    assert trainer.policy_version == 0 and ctl._buffer.released.get("untrainable_group", 0) >= 16


async def _const():
    return 0.5


def test_async_loop_config_derives_window_and_bound():
    from torchtitan_b200.experiments.rl import AsyncLoopConfig

    c = AsyncLoopConfig(num_prompts_per_train_step=8, target_offpolicy_steps=3, window_fraction=0.3)
    assert (c.max_active_rollout_groups, c.window_size, c.max_offpolicy_steps) == (32, 9, (32 + 9 - 2) // 8)
    strict = AsyncLoopConfig(num_prompts_per_train_step=8, target_offpolicy_steps=3, window_fraction=None)
    assert strict.window_size == 1 and strict.max_offpolicy_steps == 3
    with pytest.warns(UserWarning):
        AsyncLoopConfig(num_prompts_per_train_step=1, target_offpolicy_steps=0, window_fraction=0.3)
    for bad in (dict(num_prompts_per_train_step=0), dict(target_offpolicy_steps=-1), dict(window_fraction=1.5)):
        with pytest.raises(ValueError):
            AsyncLoopConfig(**bad)


# ---------------------------------------------------------------------------------------------------------- examples
def test_alphabet_sort_example():
    from torchtitan_b200.experiments.rl import Rollout, RolloutStatus
    from torchtitan_b200.experiments.rl.examples.alphabet_sort import (AlphabetSortDataset, AlphabetSortEnv,
                                                                       RewardAlphabetSort, score_sorted_list)

    ds = AlphabetSortDataset(AlphabetSortDataset.Config(seed=7, max_turns=3))
    a = [next(ds) for _ in range(3)]
    state = ds.state_dict()
    b = next(ds)
    again = AlphabetSortDataset(AlphabetSortDataset.Config(seed=7, max_turns=3))
    assert [next(again) for _ in range(3)] == a
    again.load_state_dict(json.loads(json.dumps(state)))                # survives a JSON round trip
    assert next(again) == b
    multi = next(s for s in (next(ds) for _ in range(50)) if len(s.new_names_per_turn) > 1)
    assert len(multi.expected_names[1]) == len(multi.new_names_per_turn[0]) + len(multi.new_names_per_turn[1])
    assert sum(n.endswith("// new name!") for n in multi.expected_names[1]) == len(multi.new_names_per_turn[1])
    assert score_sorted_list("<alphabetical_sorted>\nAnaB\nMarcC\n</alphabetical_sorted>", expected_names=("AnaB", "MarcC"),
                             xml_tag="alphabetical_sorted") == 1.0
    swapped = score_sorted_list("<alphabetical_sorted>MarcC\nAnaB</alphabetical_sorted>", expected_names=("AnaB", "MarcC"),
                                xml_tag="alphabetical_sorted")
    assert 0 < swapped < 1 and score_sorted_list("no block", expected_names=("x",), xml_tag="alphabetical_sorted") == 0

    async def go():
        env = AlphabetSortEnv(env_input=multi)
        first = await env.init()
        assert "alphabetical_sorted" in first.init_prompt_messages[0]["content"]
        step = await env.step({"role": "assistant", "content": "x"})
        assert not step.done and "combined_alphabetical_sorted" in step.env_messages[0]["content"]
        turns = []
        for i, names in enumerate(multi.expected_names):
            tag = "alphabetical_sorted" if i == 0 else "combined_alphabetical_sorted"
            t = _turn(0, 0, i, [1], [2])
            t.completion_message = {"role": "assistant", "content": f"<{tag}>\n" + "\n".join(names) + f"\n</{tag}>"}
            turns.append(t)
        perfect = Rollout(group_id=0, rollout_id=0, status=RolloutStatus.COMPLETED, turns=turns)
        fn = RewardAlphabetSort()
        assert await fn(perfect, multi) == pytest.approx(1.0)
        perfect.turns = turns[:1]                                       # stopped early: the missing turns score 0
        assert await fn(perfect, multi) == pytest.approx(1.0 / len(multi.expected_names))

    run(go())


def test_math_answer_example(tmp_path):
    from torchtitan_b200.experiments.rl.examples.math_answer import (MathDataset, extract_final_answer, normalize_answer,
                                                                     score_math_response)

    assert score_math_response("work\nAnswer: $34$", "34") == 1.0
    assert score_math_response("thus \\boxed{\\frac{1}{2}}", "0.5") == 1.0
    assert score_math_response("Answer: 1,234.", "1234") == 1.0
    assert score_math_response("Answer: \\boxed{12\\text{ cm}}", "12") == 1.0
    assert score_math_response("Answer: x+1", "x + 1") == 1.0
    assert score_math_response("Answer: 35", "34") == 0.0 and score_math_response("no marker 34", "34") == 0.0
    assert extract_final_answer("Answer: 1\nmore\nAnswer: 2") == "2" and extract_final_answer("\\boxed{a{b}c}") == "a{b}c"
    assert normalize_answer(" $ \\left( 3 \\right) $ ") == "(3)"
    ds = MathDataset(MathDataset.Config(seed=1, num_samples=3))
    first = [next(ds) for _ in range(3)]
    assert [next(ds) for _ in range(3)] == first                        # a fixed evaluation set cycles
    a, op, b, c = __import__("re").search(r"\((\d+) (.) (\d+)\) \* (\d+)", first[0].prompt).groups()
    assert str(eval(f"({a}{op}{b})*{c}")) == first[0].ground_truth
    path = tmp_path / "q.jsonl"
    path.write_text('{"prompt": "1+1?", "answer": 2}\n')
    assert next(MathDataset(MathDataset.Config(path=str(path)))).ground_truth == "2"


# --------------------------------------------------------------------------------------------------------------- job
def _job_args(folder, steps=2):
    return ["--module", "rl", "--config", "rl_grpo_debug_alphabet_sort", "--trainer.dump_folder", folder,
            "--controller.dump_folder", folder, "--trainer.training.mixed_precision_param", "float32",
            "--trainer.debug.no-enable_structured_logging", "--trainer.debug.seed", "0",
            "--controller.sampling.max_tokens", "6", "--controller.async_loop.num_training_steps", str(steps),
            "--controller.async_loop.batcher.batch.seq_len", "512", "--controller.async_loop.validation.num_samples", "1"]


def _run_job(rank, world, folder, out_path):
    from torchtitan_b200.config import ConfigManager

    job = ConfigManager().parse_args(_job_args(folder)).build()
    result = job.run()
    if rank == 0:
        hist = [h for h in job.controller.metrics.history if "loss/mean" in h]
        torch.save({"steps": [h["step"] for h in hist], "version": job.trainer.policy_version,
                    "dp": job.controller.dp_degree, "post": result["post"]}, out_path)
    else:
        assert result is None and job.trainer.policy_version == 2          # the followers stepped with the leader
    job.close()


def test_rl_job_from_the_config_registry(tmp_path, world=2):
    """The registered debug job end to end on two training ranks: the controller runs on rank 0 and the other rank
    follows its forward / backward and optimizer calls on its own column of the microbatch grid.  (The single-rank
    job is what ``test_rl_job_with_own_copy_generators_in_threads`` runs.)"""
    from tests.dist_utils import run_distributed

    out = str(tmp_path / "out.pt")
    run_distributed(_run_job, world, str(tmp_path / "job"), out)
    got = torch.load(out)
    assert got["steps"] == [1, 2] and got["version"] == 2 and got["dp"] == world
    assert "validation/rollout_reward/_mean" in got["post"]


def test_rl_job_config_validation():
    from torchtitan_b200.config import ConfigManager
    from torchtitan_b200.experiments.rl import config_registry as reg

    cfg = ConfigManager().parse_args(_job_args("/tmp/unused"))
    assert cfg.trainer.training.max_context_length == 512 and cfg.trainer.training.num_tokens_per_microbatch_per_dp_rank == 1024
    assert cfg.generator.threaded is False and cfg.controller.trainer_in_thread is False     # shared weights: no threads
    assert cfg.controller.rollouter.token_env.max_rollout_tokens == 511
    assert cfg.trainer.model.converters == ["lm_head_cast"]
    two = reg.rl_grpo_qwen3_0_6b_async_two_generators()
    two.validate()
    assert two.generator.threaded and two.controller.async_loop.max_offpolicy_steps >= 3
    dapo = reg.rl_dapo_qwen3_4b_math_8k()
    assert dapo.ratio_clip_high > dapo.ratio_clip_low and dapo.controller.rollouter.advantage.should_std_normalize
    tp = reg.rl_grpo_debug_alphabet_sort()
    tp.trainer.parallelism.tensor_parallel_degree = 2
    with pytest.raises(ValueError, match="data parallelism"):
        tp.validate()
    bad = reg.rl_grpo_debug_alphabet_sort()
    bad.num_generators = 2
    with pytest.raises(ValueError, match="share_weights"):
        bad.validate()
    assert reg.rl_grpo_qwen3_0_6b_alphabet_sort_batch_invariant().controller.async_loop.batcher.per_sample_pad_multiple == 128


def test_lm_head_cast_converter_keeps_logits_in_fp32():
    from torchtitan_b200.components.quantization import apply_converters
    from torchtitan_b200.experiments.rl.cast_linear import CastLinear
    from torchtitan_b200.models import get_model_spec

    spec = get_model_spec("llama3", "debugmodel")
    apply_converters(spec.model, ["lm_head_cast"])
    model = spec.model.build()
    model.init_states(seed=0)
    casts = [n for n, x in model.named_modules() if isinstance(x, CastLinear)]
    assert casts == ["lm_head"]
    ref = model(torch.tensor([1, 2, 3]))
    low = model.bfloat16()(torch.tensor([1, 2, 3]))
    assert low.dtype == torch.float32 and model.lm_head.weight.dtype == torch.bfloat16
    assert torch.allclose(low, ref, atol=0.15)
    with pytest.raises(ValueError, match="lm_head"):
        apply_converters(get_model_spec("llama3", "debugmodel").model.layers[0], ["lm_head_cast"])


def test_generate_cli_and_hf_weight_loading(tmp_path):
    """``load_hf_into`` fills a built model from a Hugging Face folder through the adapter, and the stand-alone
    generator of a registered job decodes several samples of one prompt together."""
    from safetensors.torch import save_file

    from torchtitan_b200.experiments.rl.generate import generate
    from torchtitan_b200.models import get_model_spec
    from torchtitan_b200.models.common.module import iter_checkpoint_slices
    from torchtitan_b200.scripts.convert_hf import load_hf_into

    spec = get_model_spec("llama3", "debugmodel")
    src = spec.model.build()
    src.init_states(seed=5)
    fused = dict(iter_checkpoint_slices(src))
    native = {}
    for k, p in src.named_parameters():
        for name, a, b in fused.get(k, [(k, None, None)]):
            native[name] = (p if a is None else p[a:b]).detach().clone()
    hf = spec.state_dict_adapter(spec.model, None).to_hf(native)
    save_file({k: v.contiguous() for k, v in hf.items()}, str(tmp_path / "model.safetensors"))
    dst = spec.model.build()
    dst.init_states(seed=6)
    assert load_hf_into(dst, spec, str(tmp_path)) == len(native)
    for (k, a), (_, b) in zip(src.named_parameters(), dst.named_parameters()):
        assert torch.equal(a, b), k
    with pytest.raises(FileNotFoundError):
        load_hf_into(dst, spec, str(tmp_path / "nowhere") if (tmp_path / "nowhere").mkdir() is None else "")
    texts = generate(["--config", "rl_grpo_debug_alphabet_sort", "--max-tokens", "5", "--num-samples", "3", "--temperature", "0",
                      "--device", "cpu"])
    assert len(texts) == 3 and texts[0] == texts[1] == texts[2]              # greedy: the samples agree
    assert generate(["--config", "rl_grpo_debug_alphabet_sort", "--max-tokens", "4", "--raw-prompt", "--prompt", "abc",
                     "--seed", "1", "--device", "cpu"]) != []
    with pytest.raises(ValueError):
        generate(["--config", "no_such_job"])


def test_search_qa_example_tool_calls_end_to_end(tmp_path):
    """A scripted generator calls the search tool, reads the passages and answers: the renderer shows the tool schema
    and parses the call, the environment retrieves in process, the rollout stays one growing-prefix sample, and the
    exact-match reward tells searched from closed-book and from retrieval-only outcomes."""
    from torchtitan_b200.components.tokenizer import ByteTokenizer
    from torchtitan_b200.experiments.rl import (ChatRenderer, Completion, Rollouter, Rubric, TokenEnv,
                                                TrainingSampleBuilder)
    from torchtitan_b200.experiments.rl.examples.search_qa import (PassageIndex, RewardExactMatch, SearchDataset, SearchEnv,
                                                                  normalize_answer)

    (tmp_path / "p.tsv").write_text("Eiffel Tower\tA wrought-iron tower in Paris, France.\n"
                                    "Great Wall\tA series of fortifications in northern China.\n"
                                    "Paris\tThe capital of France.\n")
    (tmp_path / "q.jsonl").write_text(json.dumps({"question": "Which city has the Eiffel Tower?", "golden_answers": ["Paris"]}) + "\n")
    idx = PassageIndex.from_file(str(tmp_path / "p.tsv"))
    assert idx.search("eiffel tower", 2)[0]["contents"].startswith("Eiffel Tower\n") and idx.search("zzz", 2) == []
    assert normalize_answer("The  Paris!") == "paris"
    with pytest.raises(ValueError):
        SearchEnv.Config()
    rend = ChatRenderer(tokenizer=ByteTokenizer())
    scripts = {0: ['<tool_call>{"name": "search", "arguments": {"query": "Eiffel Tower city"}}</tool_call><|im_end|>', "Paris<|im_end|>"],
               1: ["Paris<|im_end|>"],                                              # closed book
               2: ['<tool_call>{"name": "search", "arguments": "{\\"query\\": \\"Eiffel Tower\\"}"}</tool_call><|im_end|>', "Lyon<|im_end|>"]}
    seen_prompts = []

    async def generate_fn(prompt_token_ids, *, request_id, routing_session_id=None, sampling_config=None):
        rollout = int(request_id.split("rollout=")[1].split("/")[0])
        turn = int(request_id.rsplit("turn=", 1)[1])
        seen_prompts.append(ByteTokenizer().decode(prompt_token_ids))
        ids = rend._encode(scripts[rollout][turn])
        return Completion(request_id=request_id, token_ids=ids, token_logprobs=[-0.1] * len(ids), finish_reason="stop")

    rollouter = Rollouter.Config(
        train_dataset=SearchDataset.Config(path=str(tmp_path / "q.jsonl")), validation_dataset=SearchDataset.Config(path=str(tmp_path / "q.jsonl")),
        rubric=Rubric.Config(reward_fns=[RewardExactMatch.Config(no_search_penalty=0.2, retrieval_score=0.1)]),
        message_env=SearchEnv.Config(passages_path=str(tmp_path / "p.tsv"), topk=2),
        token_env=TokenEnv.Config(max_num_turns=4)).build()
    sample = rollouter.get_training_sample()
    group = run(rollouter.run_group_rollouts(generate_fn=generate_fn, sample=sample, group_id=0, group_size=3, sampling=None,
                                             renderer=rend))
    r0, r1, r2 = group.rollouts
    assert [len(r.turns) for r in group.rollouts] == [2, 1, 2] and all(r.status.value == "completed" for r in group.rollouts)
    assert '"name": "search"' in seen_prompts[0] and "You may call these tools" in seen_prompts[0]
    tool_msg = r0.turns[0].env_messages[0]
    assert tool_msg["role"] == "tool" and "Doc 1(Title: Eiffel Tower)" in tool_msg["content"] and "Paris" in tool_msg["content"]
    assert r2.turns[0].env_messages[0]["content"].startswith("Doc 1(Title: Eiffel Tower)")     # arguments given as a JSON string
    assert [r.reward for r in group.rollouts] == [1.0, 0.8, 0.1]
    assert sum(r.advantage for r in group.rollouts) == pytest.approx(0.0)
    samples = TrainingSampleBuilder().build_from_group(rollout_group=group).training_samples
    assert len(samples) == 3                                                          # every rollout stayed one growing prefix
    two_turn = samples[0]
    text = ByteTokenizer().decode(two_turn.token_ids)
    assert text.count("<|im_start|>tool") == 1 and text.endswith("Paris<|im_end|>")
    trained = ByteTokenizer().decode([t for t, m_ in zip(two_turn.token_ids, two_turn.loss_mask) if m_])
    assert trained.startswith("<tool_call>") and trained.endswith("Paris<|im_end|>") and "Doc 1" not in trained


def test_rl_job_with_own_copy_generators_in_threads(tmp_path):
    """Two generator replicas with their own weights decode in worker threads while the trainer trains in another; a
    pull copies the trainer's parameters into each replica and stamps the version."""
    from torchtitan_b200.config import ConfigManager

    args = _job_args(str(tmp_path), steps=3) + ["--no-share_weights", "--num_generators", "2",
                                                "--controller.async_loop.target_offpolicy_steps", "2",
                                                # all rewards are 0 here (no gradient): weight decay still moves the weights
                                                "--trainer.optimizer.weight_decay", "0.5", "--trainer.optimizer.lr", "1e-2"]
    cfg = ConfigManager().parse_args(args)
    assert cfg.generator.threaded and cfg.controller.trainer_in_thread
    job = cfg.build()
    gens = job.generators
    assert len(gens) == 2 and gens[0].model is not job.forge.model and gens[0].model is not gens[1].model
    first = {n: p.detach().clone() for n, p in gens[1].model.named_parameters()}
    out = job.run()
    assert job.trainer.policy_version == 3 and [g.policy_version for g in gens] == [3, 3]
    assert any(not torch.equal(p, first[n]) for n, p in gens[1].model.named_parameters())     # the pulls brought new weights
    src = dict(job.forge.model.named_parameters())
    for g in gens:                                          # after the last pull the replicas hold the trainer's weights
        for name, p in g.model.named_parameters():
            assert torch.equal(p, src[name].to(p.dtype)), name
    assert all(g.steps > 0 for g in gens)                   # the router used both replicas
    hist = [h for h in job.controller.metrics.history if "loss/mean" in h]
    assert [h["step"] for h in hist] == [1, 2, 3] and all(h["policy_age_max"] <= cfg.controller.async_loop.max_offpolicy_steps for h in hist)
    assert "validation/rollout_reward/_mean" in out["post"]
    job.close()


def test_rl_job_checkpoints_and_resumes(tmp_path):
    """Checkpoints at the trainer's interval carry the policy version and the datasets' positions: a second job on the
    same folder continues at the saved version, draws the next prompts of the stream and only runs the steps left."""
    from torchtitan_b200.config import ConfigManager

    def build(steps):
        return ConfigManager().parse_args(_job_args(str(tmp_path), steps=steps) + [
            "--trainer.checkpoint.enable", "--trainer.checkpoint.interval", "1", "--trainer.checkpoint.no-last_save_model_only"]).build()

    first = build(2)
    first.run()
    assert first.trainer.policy_version == 2
    position = first.controller.rollouter.dataset_state()
    first.close()
    state = json.loads((tmp_path / "checkpoint" / "rl_state.json").read_text())
    assert state["policy_version"] == 2 and "train" in state["datasets"]
    assert (tmp_path / "checkpoint" / "step-2" / ".metadata").exists()
    second = build(3)
    assert second.trainer.policy_version == 2 and second.controller.start_step == 2 and second.generators[0].policy_version == 2
    resumed_at = second.controller.rollouter.dataset_state()["train"]["rng_state"]
    assert json.loads(json.dumps(resumed_at)) == json.loads(json.dumps(state["datasets"]["train"]["rng_state"]))
    second.run()
    hist = [h["step"] for h in second.controller.metrics.history if "loss/mean" in h]
    assert hist == [3] and second.trainer.policy_version == 3 and position is not None
    second.close()


def test_renderer_with_a_tokenizer_chat_template_rerenders_between_turns():
    """With the tokenizer's own Jinja template the renderer cannot bridge turns as tokens: the token environment
    re-renders the conversation, and a template that drops earlier reasoning breaks the prefix, so the rollout packs
    into two training samples instead of one."""
    from torchtitan_b200.components.tokenizer import ByteTokenizer
    from torchtitan_b200.experiments.rl import ChatRenderer, TokenEnv, TrainingSampleBuilder

    tok = ByteTokenizer()
    tok.chat_template = ("{% for m in messages %}[{{ m['role'] }}]{{ m['content'] }}\\n{% endfor %}"
                         "{% if add_generation_prompt %}[assistant]{% endif %}")
    rend = ChatRenderer(tokenizer=tok)
    ids = rend.render_ids(messages=[{"role": "user", "content": "hi"}])
    assert tok.decode(ids) == "[user]hi\\n[assistant]"
    assert rend.bridge_to_next_turn(previous_prompt_ids=ids, previous_completion_ids=[1], new_messages=[]) is None

    async def go():
        env = TokenEnv(message_env=_EchoEnv(turns=2), renderer=rend)
        first = await env.init()
        c1 = _completion(rend, "<think>secret</think>one")
        second = await env.step(c1)
        return first, c1, second

    first, c1, second = run(go())
    text = tok.decode(second.next_prompt_token_ids)
    assert text == "[user]hi\\n[assistant]one\\n[user]again\\n[assistant]"          # the reasoning is not in the history
    turns = [_turn(0, 0, 0, first.next_prompt_token_ids, c1.token_ids), _turn(0, 0, 1, second.next_prompt_token_ids, rend._encode("two"))]
    samples = TrainingSampleBuilder().rollout_to_training_samples(_rollout(0, 0, turns, 1.0, 0.5))
    assert len(samples) == 2 and samples[1].rollout_id.turn_id == 1


def test_place_model_keeps_buffer_dtypes():
    """Parameters go to bf16, the fp32 rotary tables stay fp32 (``model.to(dtype=...)`` would cast them and the kernels
    that read them refuse that), and the engine decodes on the result."""
    from torchtitan_b200.experiments.rl import GenerationEngine, SamplingConfig
    from torchtitan_b200.experiments.rl.engine import place_model_

    _, model = _tiny_llama()
    place_model_(model, torch.device("cpu"), torch.bfloat16)
    assert all(p.dtype == torch.bfloat16 for p in model.parameters())
    tables = [b for n, b in model.named_buffers() if n.endswith("rope.cache")]
    assert tables and all(b.dtype == torch.float32 for b in tables)

    async def go():
        eng = GenerationEngine(GenerationEngine.Config(threaded=False), model=model)
        out = await eng.generate([3, 4, 5], request_id="x", sampling_config=SamplingConfig(temperature=0.0, max_tokens=4))
        await eng.close()
        return out

    assert len(run(go()).token_ids) == 4


def test_data_parallel_engine_spreads_requests_and_keeps_sessions_together():
    from torchtitan_b200.experiments.rl import (DataParallelEngine, GenerationEngine, InterGeneratorRouter,
                                                IntraGeneratorRouter, LeastLoadedRoutingStrategy, SamplingConfig)

    _, model = _tiny_llama()
    greedy = SamplingConfig(temperature=0.0, max_tokens=3)

    async def go():
        ranks = [GenerationEngine(GenerationEngine.Config(threaded=False), model=model) for _ in range(2)]
        dp = DataParallelEngine(ranks, IntraGeneratorRouter.Config(strategy=LeastLoadedRoutingStrategy.Config()))
        out = await asyncio.gather(*(dp.generate([i + 1, 2], request_id=f"q{i}", sampling_config=greedy) for i in range(6)))
        assert all(len(c.token_ids) == 3 for c in out) and dp.router.loads() == [0, 0]
        assert ranks[0].tokens_generated > 0 and ranks[1].tokens_generated > 0
        sticky = DataParallelEngine([GenerationEngine(GenerationEngine.Config(threaded=False), model=model) for _ in range(2)])
        for turn in range(3):
            await sticky.generate([7, 8, turn + 1], request_id=f"s/turn={turn}", routing_session_id="s", sampling_config=greedy)
        assert sorted(e.tokens_generated for e in sticky.engines) == [0, 9]          # one rank served the whole session
        front = InterGeneratorRouter(generators=[dp, sticky])                          # layer one in front of layer two
        await front.generate([3, 4], request_id="f0", sampling_config=greedy)
        await front.pull_model_state_dict(4)
        assert dp.policy_version == 4 and all(e.policy_version == 4 for e in sticky.engines)
        await front.close_generators()

    run(go())
    with pytest.raises(ValueError):
        DataParallelEngine([GenerationEngine(model=model)])


def test_engine_leaves_the_routers_load_counters_alone():
    """Generation on a model shared with the trainer must not feed the expert-load statistics that drive the
    trainer's balancing bias."""
    from torchtitan_b200.experiments.rl import GenerationEngine, SamplingConfig
    from torchtitan_b200.models import get_model_spec

    spec = get_model_spec("qwen3", "debugmodel_moe_tiny")
    model = spec.model.build()
    model.init_states(seed=0)
    moes = [m_ for m_ in model.modules() if hasattr(m_, "tokens_per_expert_E")]
    assert moes
    for m_ in moes:
        m_.tokens_per_expert_E.fill_(3.0)

    async def go():
        eng = GenerationEngine(GenerationEngine.Config(threaded=False), model=model)
        out = await eng.generate([1, 2, 3, 4], request_id="x", sampling_config=SamplingConfig(temperature=0.0, max_tokens=3))
        await eng.close()
        return out

    assert len(run(go()).token_ids) == 3
    assert all(bool((m_.tokens_per_expert_E == 3.0).all()) for m_ in moes)


def test_engine_stops_at_the_models_context():
    from torchtitan_b200.experiments.rl import GenerationEngine, SamplingConfig

    _, model = _tiny_llama()
    ctx = model.config.max_context_length
    model.config.max_context_length = 12           # pretend the tables end here

    async def go():
        eng = GenerationEngine(GenerationEngine.Config(threaded=False), model=model)
        out = await eng.generate(list(range(1, 9)), request_id="a", sampling_config=SamplingConfig(temperature=0.0, max_tokens=50))
        with pytest.raises(ValueError, match="context"):
            await eng.generate(list(range(1, 14)), request_id="b")
        await eng.close()
        return out

    try:
        out = run(go())
    finally:
        model.config.max_context_length = ctx
    assert out.finish_reason == "length" and len(out.token_ids) == 12 - 8      # rows 0..11 were fed or produced
