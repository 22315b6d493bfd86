"""OaCli precedence: record defaults < YAML file < arguments the user typed (Source/Public/Oa/Core/Cli.h:1-140)."""
from dataclasses import dataclass, field

from oa_b200.utils.cli import OaCli


@dataclass
class Cfg:
    Lr: float = 3e-4
    Data: str = "none"
    Steps: int = 100
    UseGraph: bool = True
    Layers: list = field(default_factory=lambda: [1, 2])
    Resume: bool = False


class Cli(OaCli):
    def __init__(self):
        super().__init__("train", "Train a model", Cfg())
        self.AddOption("--lr", "Lr", "learning rate")
        self.AddOption("--data,-d", "Data", "data file")
        self.AddOption("--steps", "Steps", "steps")
        self.AddOption("--graph", "UseGraph", "capture the step")
        self.AddOption("--layers", "Layers", "layer ids")
        self.AddFlag("--resume", "Resume", "resume from the last checkpoint")

    def Validate(self):
        return "steps must be positive" if self.Cfg.Steps <= 0 else None


def test_defaults_then_yaml_then_typed_arguments(tmp_path):
    y = tmp_path / "c.yaml"
    y.write_text("lr: 0.01\nsteps: 7\ndata: from_yaml\nunknown_key: 1\n")
    c = Cli()
    assert c.Parse(["train"]) and c.Cfg == Cfg()
    c = Cli()
    assert c.Parse(["train", "--config", str(y)])
    assert (c.Cfg.Lr, c.Cfg.Steps, c.Cfg.Data, c.Cfg.UseGraph) == (0.01, 7, "from_yaml", True)
    c = Cli()
    assert c.Parse(["train", f"--config={y}", "--steps", "9", "-d", "typed", "--no-graph", "--layers", "4", "5", "6", "--resume", "-v", "2"])
    assert (c.Cfg.Lr, c.Cfg.Steps, c.Cfg.Data, c.Cfg.UseGraph, c.Cfg.Layers, c.Cfg.Resume, c.Verbose) == (0.01, 9, "typed", False, [4, 5, 6], True, 2)
    assert c.ConfigPath == str(y)


def test_errors_do_not_raise(tmp_path, capsys):
    c = Cli()
    assert not c.Parse(["train", "--steps", "many"]) and c.Error
    c = Cli()
    assert not c.Parse(["train", "--steps", "0"]) and c.Error == "steps must be positive"
    c = Cli()
    assert c.Parse(["train", "-c", str(tmp_path / "missing.yaml"), "--lr", "0.5"]) and c.Cfg.Lr == 0.5      # warns, keeps defaults
    assert "YAML load failed" in c.Error
    assert "--lr" in Cli().Usage() and "--help-all" in Cli().Usage()
    capsys.readouterr()


def test_enum_string_forms():
    """<Type>ToString / <Type>FromString of the generated type header (Source/Public/Oa/Core/Type.gen.h:15-66)."""
    import oa
    assert oa.OaScalarTypeToString(oa.OaScalarType.BFloat16) == "BFloat16" and oa.OaScalarTypeFromString("bfloat16") == oa.OaScalarType.BFloat16
    assert oa.OaPrecisionFromString("BF16") == oa.OaPrecision.BF16 and oa.OaPrecisionToString(0) == "FP32"
    assert oa.OaPrecisionFromString("no such precision") == oa.OaPrecision.FP32            # unknown text: the first member
    assert oa.OaMatMulPrecisionFromString(" fp32 ") == oa.OaMatMulPrecision.Fp32
    assert oa.OaEnumFromString(oa.OaStatusCode, "notfound") == oa.OaStatusCode.NotFound and oa.OaEnumToString(oa.OaStatusCode.Ok) == "Ok"
