"""``axolotl`` command line: preprocess / train / evaluate / inference / merge-lora /
merge-sharded-fsdp-weights / fetch / quantize / config-schema / vllm-serve / chat.

Every top-level config key is also accepted as ``--key value`` (nested: ``--parent__child``), like
the reference CLI (src/axolotl/cli/main.py:42-501, src/axolotl/cli/utils/args.py:191-219).
``train`` re-launches itself under ``torchrun`` when several GPUs are visible
(``--launcher torchrun|python``, ``--num-processes N``).
"""
from __future__ import annotations

import json
import os
import shutil
import subprocess
import sys

import click

from ..utils.logging import get_logger

LOG = get_logger(__name__)
CONTEXT = dict(ignore_unknown_options=True, allow_extra_args=True)


def _extra_to_overrides(args):
    """['--lora_r', '16', '--bf16', '--no-sample_packing', '--a=b'] -> dict"""
    out, i = {}, 0
    while i < len(args):
        a = args[i]
        if not a.startswith("--"):
            i += 1
            continue
        key = a[2:]
        if "=" in key:
            key, val = key.split("=", 1)
            out[key.replace("-", "_")] = val
            i += 1
            continue
        if key.startswith("no-") or key.startswith("no_"):
            out[key[3:].replace("-", "_")] = False
            i += 1
            continue
        if i + 1 < len(args) and not args[i + 1].startswith("--"):
            out[key.replace("-", "_")] = args[i + 1]
            i += 2
        else:
            out[key.replace("-", "_")] = True
            i += 1
    return out


def _wants_ray(config, ctx) -> bool:
    """``use_ray: true`` in the YAML or ``--use-ray`` on the command line (read before any process group exists)."""
    ov = _extra_to_overrides(ctx.args)
    if "use_ray" in ov:
        return str(ov["use_ray"]).lower() in ("1", "true", "yes")
    try:
        import yaml as _yaml

        from ..config.load import fetch_config

        with open(fetch_config(config), encoding="utf-8") as fh:
            return bool((_yaml.safe_load(fh) or {}).get("use_ray"))
    except (OSError, ValueError):
        return False


def _load(config, ctx, **forced):
    from ..config.load import load_cfg

    ov = _extra_to_overrides(ctx.args)
    ov.update(forced)
    return load_cfg(config, **ov)


@click.group()
@click.version_option(package_name=None, version="0.1.0", prog_name="axolotl (b200)")
def cli():
    """Blackwell-native fine-tuning with the axolotl configuration surface."""


@cli.command(context_settings=CONTEXT)
@click.argument("config")
@click.option("--debug", is_flag=True, help="print a few tokenised samples with their label mask")
@click.option("--debug-num-examples", default=3)
@click.option("--cloud", type=click.Path(exists=True), default=None, help="cloud YAML: run the command on that provider")
@click.option("--no-cloud", is_flag=True, hidden=True)
@click.pass_context
def preprocess(ctx, config, debug, debug_num_examples, cloud, no_cloud):
    """Tokenise + cache the datasets of CONFIG (CPU only)."""
    if cloud and not no_cloud:
        from .launchers import run_in_cloud

        return run_in_cloud("preprocess", cloud, config)
    os.environ["AXOLOTL_IS_PREPROCESS"] = "1"
    cfg = _load(config, ctx, is_preprocess=True)
    if not cfg.get("dataset_prepared_path"):
        cfg["dataset_prepared_path"] = "last_run_prepared"
    from ..data.loading import load_datasets

    meta = load_datasets(cfg, preprocess=True)
    click.echo(f"prepared {len(meta.train)} training samples ({meta.train.total_tokens()} tokens) under "
               f"{cfg['dataset_prepared_path']}")
    if debug:
        from ..data.debug import print_samples

        print_samples(meta.train, cfg, debug_num_examples)


def _visible_gpus():
    try:
        import torch

        return torch.cuda.device_count()
    except Exception:
        return 0


@cli.command(context_settings=CONTEXT)
@click.argument("config")
@click.option("--launcher", type=click.Choice(["torchrun", "python", "accelerate"]), default=None)
@click.option("--num-processes", type=int, default=None)
@click.option("--main-process-port", type=int, default=29500)
@click.option("--sweep", type=click.Path(exists=True), default=None, help="YAML with lists of values to grid over")
@click.option("--cloud", type=click.Path(exists=True), default=None, help="cloud YAML: run the command on that provider")
@click.pass_context
def train(ctx, config, launcher, num_processes, main_process_port, sweep, cloud):
    """Train (or fine-tune) the model described by CONFIG."""
    if cloud:
        from .launchers import run_in_cloud

        return run_in_cloud("train", cloud, config, launcher=launcher or "torchrun", launcher_args=list(ctx.args),
                            num_processes=num_processes)
    if _wants_ray(config, ctx):
        from ..config.load import apply_overrides, fetch_config
        from .launchers import train_with_ray
        import yaml as _yaml

        raw = apply_overrides(_yaml.safe_load(open(fetch_config(config), encoding="utf-8")) or {}, _extra_to_overrides(ctx.args))
        return train_with_ray(_load(config, ctx), raw)
    if sweep:
        from .sweeps import expand_sweep

        for i, path in enumerate(expand_sweep(config, sweep)):
            click.echo(f"[sweep {i}] {path}")
            rc = subprocess.call([sys.executable, "-m", "axolotl_b200.cli.main", "train", path, *ctx.args])
            if rc:
                sys.exit(rc)
        return
    n = num_processes or int(os.environ.get("WORLD_SIZE", 0)) or _visible_gpus() or 1
    already = "RANK" in os.environ
    if launcher == "accelerate":
        LOG.warning("the accelerate launcher is served by torchrun on axolotl_b200")
        launcher = "torchrun"
    if launcher is None:
        launcher = "torchrun" if (n > 1 and not already) else "python"
    if launcher == "torchrun" and not already:
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}",
               "--master-addr", os.environ.get("MASTER_ADDR", "127.0.0.1"), "--master-port", str(main_process_port),
               "-m", "axolotl_b200.cli.main", "train", config, "--launcher", "python", *ctx.args]
        os.execvpe(cmd[0], cmd, os.environ)
    cfg = _load(config, ctx)
    from ..train.run import train as run_train

    run_train(cfg)


@cli.command(context_settings=CONTEXT)
@click.argument("config")
@click.pass_context
def evaluate(ctx, config):
    """Evaluation loss / perplexity on the validation split or test_datasets of CONFIG."""
    cfg = _load(config, ctx)
    from ..train.evaluate import evaluate as run_eval

    click.echo(json.dumps(run_eval(cfg)))


@cli.command(context_settings=CONTEXT)
@click.argument("config")
@click.option("--prompt", default=None, help="prompt text (stdin when omitted)")
@click.option("--max-new-tokens", default=64)
@click.option("--temperature", default=0.0)
@click.option("--lora-model-dir", default=None)
@click.option("--gradio", is_flag=True, help="serve a browser interface instead of answering one prompt")
@click.pass_context
def inference(ctx, config, prompt, max_new_tokens, temperature, lora_model_dir, gradio):
    """Generate from the (optionally adapter-augmented) model of CONFIG."""
    forced = {"lora_model_dir": lora_model_dir} if lora_model_dir else {}
    cfg = _load(config, ctx, **forced)
    if gradio:
        from .gradio_ui import launch

        try:
            return launch(cfg)
        except RuntimeError as e:
            raise click.ClickException(str(e))
    from ..train.evaluate import generate_text

    text = prompt if prompt is not None else sys.stdin.read()
    click.echo(generate_text(cfg, text, max_new_tokens=max_new_tokens, temperature=temperature))


@cli.command("chat", context_settings=CONTEXT)
@click.argument("config")
@click.option("--system", default=None, help="system prompt")
@click.option("--max-new-tokens", default=256)
@click.option("--temperature", default=0.7)
@click.option("--lora-model-dir", default=None)
@click.pass_context
def chat(ctx, config, system, max_new_tokens, temperature, lora_model_dir):
    """Interactive multi-turn chat with the model (and adapter) of CONFIG."""
    forced = {"lora_model_dir": lora_model_dir} if lora_model_dir else {}
    cfg = _load(config, ctx, **forced)
    from .chat import run_repl

    run_repl(cfg, system, max_new_tokens, temperature, echo=click.echo)


@cli.command("merge-lora", context_settings=CONTEXT)
@click.argument("config")
@click.option("--lora-model-dir", default=None)
@click.option("--output-dir", default=None)
@click.pass_context
def merge_lora(ctx, config, lora_model_dir, output_dir):
    """Fold the trained adapter into the base weights -> <output_dir>/merged."""
    cfg = _load(config, ctx, load_in_4bit=False, load_in_8bit=False)
    adapter = lora_model_dir or cfg.get("lora_model_dir") or cfg["output_dir"]
    out = os.path.join(output_dir or cfg["output_dir"], "merged")
    base = cfg.get("base_model")
    if not base or not os.path.isdir(base):
        raise click.ClickException("merge-lora needs `base_model` to be a local HF checkpoint directory")
    from ..io.merge import merge_lora_sharded

    res = merge_lora_sharded(base, adapter, out)
    click.echo(f"merged {res['merged']} modules across {res['files']} shard file(s) into {out}")


@cli.command("merge-sharded-fsdp-weights", context_settings=CONTEXT)
@click.argument("config")
@click.pass_context
def merge_sharded(ctx, config):
    """Combine per-rank shard files under <output_dir>/pytorch_model_fsdp_0 into one HF checkpoint."""
    cfg = _load(config, ctx)
    from ..io.merge import merge_sharded_fsdp_weights

    src = os.path.join(cfg["output_dir"], "pytorch_model_fsdp_0")
    files = merge_sharded_fsdp_weights(src, os.path.join(cfg["output_dir"], "merged"))
    click.echo(f"wrote {len(files)} file(s) to {os.path.join(cfg['output_dir'], 'merged')}")


@cli.command(context_settings=CONTEXT)
@click.argument("config")
@click.option("--output-dir", default=None)
@click.pass_context
def quantize(ctx, config, output_dir):
    """Post-training quantisation of MoE expert weights to NVFP4 (frozen-expert format)."""
    cfg = _load(config, ctx)
    from ..train.run import build_model
    from ..ops.grouped import quantize_experts_nvfp4_
    from ..io.hf import save_pretrained
    import torch

    model = build_model(cfg, torch.device("cpu"))
    quantize_experts_nvfp4_(model)
    out = output_dir or os.path.join(cfg["output_dir"], "quantized")
    save_pretrained(model, out)
    click.echo(f"wrote NVFP4 checkpoint to {out}")


@cli.command()
@click.argument("directory", type=click.Choice(["examples", "deepspeed_configs"]))
@click.option("--dest", default=None)
def fetch(directory, dest):
    """Copy the bundled example configs into the working directory."""
    if directory == "deepspeed_configs":
        raise click.ClickException("DeepSpeed is not used by axolotl_b200; there are no DeepSpeed configs to fetch")
    src = os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "examples")
    dst = dest or directory
    shutil.copytree(src, dst, dirs_exist_ok=True)
    click.echo(f"copied examples to {dst}")


@cli.command("config-schema")
@click.option("--format", "output_format", type=click.Choice(["json", "yaml"]), default="json")
@click.option("--field", default=None, help="show the schema of one field only")
def config_schema(output_format, field):
    """Dump the JSON schema of the configuration (all keys, types, defaults)."""
    from ..config.schema import AxolotlConfig

    schema = AxolotlConfig.model_json_schema()
    if field:
        props = schema.get("properties", {})
        if field not in props:
            match = [k for k in props if k.lower() == field.lower()]
            if not match:
                raise click.BadParameter(f"unknown field {field!r}; omit --field to dump the full schema")
            field = match[0]
        schema = {field: props[field]}
    if output_format == "yaml":
        import yaml

        click.echo(yaml.dump(schema, default_flow_style=False, sort_keys=False))
    else:
        click.echo(json.dumps(schema, indent=2))


@cli.command("agent-docs")
@click.argument("topic", required=False, default=None)
@click.option("--list", "list_topics", is_flag=True, help="list the available topics")
def agent_docs(topic, list_topics):
    """Print the bundled reference notes written for coding agents (no network needed)."""
    root = os.path.join(os.path.dirname(os.path.abspath(__file__)), "agent_docs")
    topics = sorted(f[:-3] for f in os.listdir(root) if f.endswith(".md"))
    if list_topics:
        for t in topics:
            with open(os.path.join(root, t + ".md")) as fh:
                click.echo(f"  {t:15s} {fh.readline().lstrip('# ').strip()}")
        return
    topic = topic or "overview"
    if topic not in topics:
        raise click.BadParameter(f"unknown topic {topic!r} (have: {', '.join(topics)})")
    with open(os.path.join(root, topic + ".md")) as fh:
        click.echo(fh.read())


@cli.command("generate-cli-config-options")
@click.option("--output", default="config_options.json", show_default=True, help="file to write")
@click.option("--check", is_flag=True, help="fail if the file on disk is stale")
def generate_cli_config_options(output, check):
    """Write the table of command-line overrides (one ``--key`` per scalar config field, with its type)."""
    from ..config.schema import AxolotlConfig

    rows = {}
    for name, info in sorted(AxolotlConfig.model_fields.items()):
        ann = str(info.annotation)
        kind = next((k for k in ("bool", "int", "float", "str") if k in ann), None)
        if kind is None or "dict" in ann or "list" in ann.lower():
            continue
        rows[name] = {"option": "--" + name.replace("_", "-"), "type": kind,
                      "default": info.default if isinstance(info.default, (bool, int, float, str, type(None))) else None}
    text = json.dumps(rows, indent=1, sort_keys=True) + "\n"
    if check:
        if not os.path.exists(output) or open(output).read() != text:
            raise click.ClickException(f"{output} is stale: run `axolotl generate-cli-config-options --output {output}`")
        click.echo(f"{output} is up to date ({len(rows)} options)")
        return
    with open(output, "w") as fh:
        fh.write(text)
    click.echo(f"wrote {len(rows)} options to {output}")


@cli.command("delinearize-llama4")
@click.argument("model")
@click.argument("output")
def delinearize_llama4(model, output):
    """Convert linearised Llama-4 expert weights back to the fused layout."""
    raise click.ClickException("Llama-4 is not among the architectures of this framework "
                               "(llama, mistral, phi3, qwen2, qwen3, granite, smollm3 and the qwen/mixtral/olmoe MoE families)")


@cli.command("vllm-serve", context_settings=CONTEXT)
@click.argument("config")
@click.pass_context
def vllm_serve(ctx, config):
    """Start the generation server that GRPO runs with ``trl.use_vllm: true`` sample from."""
    from ..config.load import load_cfg
    from ..rl.vllm_server import serve

    cfg = load_cfg(config, **_extra_to_overrides(ctx.args))
    try:
        serve(cfg)
    except RuntimeError as exc:
        raise click.ClickException(str(exc)) from exc


def main():
    cli()


if __name__ == "__main__":
    main()
