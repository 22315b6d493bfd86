"""The reference's NLP tutorials as one GPU test per architecture (Tutorial/Ml/Nlp/TutorialNlpByteTransformerAg.cpp:142-251,
Tutorial/Py/Ml/Nlp/_nlp_common.py:256-283): train the suite recipe for 300 AdamW steps on CUDA through OaItTraining with the
step captured as a program, pass the accuracy gate (> 30 % for Transformer / MoE / Mamba-3, > 50 % for GRU on characters),
generate from the prompt, save one `.oam` file, load it into a FRESH model + optimizer, and find the same accuracy
(within 0.5 %), the same generation, the same step counter and the same next optimizer step."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _engine():
    from oa_b200.core.types import OaPrecision
    from oa_b200.runtime.engine import OaEngineConfig, OaInitComputeEngine
    assert OaInitComputeEngine(OaEngineConfig(Precision=OaPrecision.FP32, DeviceIndex=0))


@pytest.mark.parametrize("arch_name,gate", [("Transformer", 0.30), ("MoeTransformer", 0.30), ("Mamba3", 0.30), ("Gru", 0.50)])
def test_tutorial_train_generate_save_reload(arch_name, gate, tmp_path):
    from oa_b200.core import fn_matrix as F
    from oa_b200.ml import fn_loss as L
    from oa_b200.ml import nlp_suite as NS
    from oa_b200.ml.autograd import OaGradientTape, OaGradNo
    from oa_b200.ml.optim import OaAdamW
    from oa_b200.ml.training import OaItTraining, OaItTrainingConfig
    from oa_b200.ops import kernels as K
    _engine()
    arch = getattr(NS.OaNlpArchitecture, arch_name)
    recipe = NS.OaNlpSuiteRecipe(arch, NS.OaNlpTokenizerKind.Char)
    B, S, steps = NS.OaNlpSuiteBatchSize, recipe.ContextLength(), 300

    def build(seed):
        F.SetRngSeed(seed)
        model = NS.OaNlpSuiteModel(recipe)
        return model, OaAdamW(model.AllParameterPtrs(), recipe.LearningRate())

    model, opt = build(NS.OaNlpSuiteRngSeed)
    sampler = NS.OaNlpSuiteSampler(recipe, B)
    dev = F._dev()
    ids = F.FromTensor(torch.empty((B, S), dtype=torch.int32, device=dev))
    tgt = F.FromTensor(torch.empty((B * S,), dtype=torch.int32, device=dev))

    def prepare():
        x, y = sampler.Next()
        ids.Tensor().copy_(x.Tensor())
        tgt.Tensor().copy_(y.Tensor().reshape(-1))

    def make_record(m, o):
        def record():
            o.ZeroGrad()
            with OaGradientTape() as tape:
                loss = L.CrossEntropy(m.Forward(ids), tgt)
                tape.Backward(loss)
            return loss
        return record

    tr = OaItTraining(opt, OaItTrainingConfig(TotalSteps=steps, BatchSize=B, SequenceLength=S, Program=True))
    losses = []
    record = make_record(model, opt)
    while not tr.IsDone():
        losses.append(tr.Step(prepare, record))
    tr.Finish()
    assert tr.Program().IsCaptured() and tr.Program().Replays >= steps - 3
    assert losses[-1] < 0.5 * losses[0], (losses[0], losses[-1])

    def accuracy(m):
        with OaGradNo():
            logits = m.Forward(ids).Tensor().float().reshape(B * S, -1)
        return (logits.argmax(1) == tgt.Tensor().long()).float().mean().item()

    acc = accuracy(model)
    assert acc > gate, f"{arch_name}: final-batch accuracy {acc:.3f} does not pass the {gate:.0%} gate"
    text = NS.OaNlpSuiteGenerate(model, sampler, source_units=80)
    assert text.startswith(NS.OaNlpSuiteGenerationPrompt) and len(text) == len(NS.OaNlpSuiteGenerationPrompt) + 80

    path = str(tmp_path / f"{recipe.ArchitectureId()}.oam")
    assert model.Save(path, opt)
    fresh, fresh_opt = build(1)                                   # different initial weights: everything must come from the file
    assert fresh.Load(path, fresh_opt)
    assert abs(accuracy(fresh) - acc) <= 0.005
    assert NS.OaNlpSuiteGenerate(fresh, sampler, source_units=80) == text
    assert fresh_opt.GetStep() == opt.GetStep() == steps
    # one more optimizer step on the same batch from both: identical parameters afterwards
    make_record(model, opt)()
    opt.Step()
    make_record(fresh, fresh_opt)()
    fresh_opt.Step()
    torch.cuda.synchronize()
    K.check_status()
    # (the embedding gradient is accumulated with floating-point atomics, so two runs of one step agree to rounding, not bit for bit)
    for a, b in zip(model.AllParameterPtrs(), fresh.AllParameterPtrs()):
        assert torch.allclose(a.Tensor(), b.Tensor(), rtol=1e-5, atol=1e-6), a.Name
