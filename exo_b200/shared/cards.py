"""Model cards: the TOML half of the checkpoint contract.

A card says what a model repository needs from the cluster (size, layers, hidden size, KV heads,
whether it may be tensor-sharded, sampling defaults, capabilities).  The schema is the reference's
(``src/exo/shared/models/model_cards.py:118-177`` and the TOMLs under
``resources/inference_model_cards``) so its card files load unchanged; ``Backend`` gains the value
``B200`` for this engine.  Cards come from three places, first hit wins: built-in resources,
the user's custom-card directory, and — for an unknown id — the repository's own ``config.json`` +
safetensors index (``fetch_card``; reference ``model_cards.py:236-262``).
"""
from __future__ import annotations

import json
import os
import tomllib
from enum import Enum
from pathlib import Path
from typing import Annotated, Any

from pydantic import AliasChoices, BaseModel, Field, PositiveInt, field_validator, model_validator

from .base import FrozenModel, Memory, ModelId
from . import constants

ReasoningDialectT = str


class Backend(str, Enum):
    MlxMetal = "MlxMetal"
    MlxCpu = "MlxCpu"
    MlxCuda = "MlxCuda"
    Vllm = "Vllm"
    B200 = "B200"


class ModelTask(str, Enum):
    TextGeneration = "TextGeneration"
    TextToImage = "TextToImage"
    ImageToImage = "ImageToImage"


class ComponentInfo(FrozenModel):
    component_name: str
    component_path: str
    storage_size: Memory
    n_layers: PositiveInt | None = None
    can_shard: bool
    safetensors_index_filename: str | None = None


class VisionCardConfig(FrozenModel):
    image_token_id: int
    model_type: str
    weights_repo: str = ""
    image_token: str | None = None
    processor_repo: str | None = None


class SamplingValues(FrozenModel):
    temperature: float | None = None
    top_p: float | None = None
    top_k: int | None = None
    min_p: float | None = None
    repetition_penalty: float | None = None
    presence_penalty: float | None = None
    frequency_penalty: float | None = None


class SamplingDefaults(SamplingValues):
    thinking: SamplingValues | None = None
    non_thinking: SamplingValues | None = None


class ModelCard(FrozenModel):
    model_id: ModelId
    storage_size: Memory
    n_layers: PositiveInt
    hidden_size: PositiveInt
    supports_tensor: bool
    num_key_value_heads: PositiveInt | None = None
    tasks: list[ModelTask]
    components: list[ComponentInfo] | None = None
    family: str = ""
    quantization: str = ""
    base_model: str = ""
    capabilities: list[str] = []
    backends: list[Backend] = Field(default_factory=lambda: list(Backend))
    reasoning_dialect: str = "none"
    context_length: int = 0
    uses_cfg: bool = False
    trust_remote_code: bool = True
    is_custom: bool = False
    vision: VisionCardConfig | None = None
    sampling_defaults: SamplingDefaults = Field(default_factory=SamplingDefaults)

    @field_validator("tasks", mode="before")
    @classmethod
    def _tasks(cls, v: list[Any]) -> list[ModelTask]:
        return [t if isinstance(t, ModelTask) else ModelTask(t) for t in v]

    @field_validator("backends", mode="before")
    @classmethod
    def _backends(cls, v: list[Any]) -> list[Backend]:
        return [b if isinstance(b, Backend) else Backend(b) for b in v]

    @field_validator("storage_size", mode="before")
    @classmethod
    def _size(cls, v: Any) -> Any:
        return {"in_bytes": v} if isinstance(v, int) else v

    @model_validator(mode="after")
    def _vision_repo(self) -> "ModelCard":
        if self.vision is not None and not self.vision.weights_repo:
            object.__setattr__(self, "vision", self.vision.model_copy(update={"weights_repo": str(self.model_id)}))
        return self

    @property
    def is_image(self) -> bool:
        return any(t in (ModelTask.TextToImage, ModelTask.ImageToImage) for t in self.tasks)

    # ---- TOML ----
    def to_toml(self) -> str:
        return dumps_toml(self.model_dump(exclude_none=True, exclude={"is_custom"}, mode="json", by_alias=False))

    def save(self, path: Path) -> None:
        path.parent.mkdir(parents=True, exist_ok=True)
        path.write_text(self.to_toml())

    @staticmethod
    def load_from_path(path: Path) -> "ModelCard":
        with open(path, "rb") as f:
            return ModelCard.model_validate(tomllib.load(f), strict=False)


def dumps_toml(d: dict[str, Any]) -> str:
    """Small TOML writer for card-shaped data (scalars, lists of scalars, nested tables, arrays of tables)."""
    def scalar(v: Any) -> str:
        if isinstance(v, bool):
            return "true" if v else "false"
        if isinstance(v, (int, float)):
            return repr(v)
        if isinstance(v, str):
            return json.dumps(v)
        if isinstance(v, list):
            return "[" + ", ".join(scalar(x) for x in v) + "]"
        raise TypeError(f"cannot encode {type(v)}")

    out: list[str] = []

    def table(prefix: str, t: dict[str, Any]) -> None:
        simple = {k: v for k, v in t.items() if not isinstance(v, dict) and not (isinstance(v, list) and v and isinstance(v[0], dict))}
        for k, v in simple.items():
            out.append(f"{k} = {scalar(v)}")
        for k, v in t.items():
            if isinstance(v, dict):
                out.append(f"\n[{prefix}{k}]")
                table(f"{prefix}{k}.", v)
            elif isinstance(v, list) and v and isinstance(v[0], dict):
                for item in v:
                    out.append(f"\n[[{prefix}{k}]]")
                    table(f"{prefix}{k}.", item)

    table("", d)
    return "\n".join(out) + "\n"


# --------------------------------------------------------------------------------------------
# HF config.json → card facts
# --------------------------------------------------------------------------------------------
TENSOR_ARCHITECTURES = {
    "LlamaForCausalLM", "MistralForCausalLM", "Qwen2ForCausalLM", "Qwen3ForCausalLM", "Qwen3MoeForCausalLM",
    "DeepseekV3ForCausalLM", "DeepseekV32ForCausalLM", "GptOssForCausalLM",
}


class ConfigData(BaseModel):
    """The few facts a card needs out of ``config.json`` (``text_config`` is unwrapped first)."""
    model_config = {"extra": "ignore"}
    architectures: list[str] | None = None
    hidden_size: Annotated[int, Field(ge=0)] | None = None
    num_key_value_heads: PositiveInt | None = None
    layer_count: int = Field(validation_alias=AliasChoices("num_hidden_layers", "num_layers", "n_layer", "n_layers",
                                                            "num_decoder_layers", "decoder_layers"))
    max_position_embeddings: int = 0
    vision: VisionCardConfig | None = None

    @property
    def supports_tensor(self) -> bool:
        return bool(self.architectures) and self.architectures[0] in TENSOR_ARCHITECTURES

    @model_validator(mode="before")
    @classmethod
    def _text_config(cls, data: dict[str, Any], info) -> dict[str, Any]:
        tc = data.get("text_config")
        if isinstance(tc, dict):
            for k in ("architectures", "hidden_size", "num_key_value_heads", "max_position_embeddings", "num_hidden_layers",
                      "num_layers", "n_layer", "n_layers", "num_decoder_layers", "decoder_layers"):
                if tc.get(k) is not None:
                    data[k] = tc[k]
        if data.get("vision_config") is not None and data.get("image_token_id") is not None:
            mid = (info.context or {}).get("model_id", "") if info is not None else ""
            data["vision"] = VisionCardConfig(image_token_id=int(data["image_token_id"]),
                                              model_type=str(data.get("model_type", "")), weights_repo=mid)
        return data


def card_from_local_dir(model_id: ModelId, path: Path) -> ModelCard:
    """Build a card from a checkpoint directory (``config.json`` + safetensors files/index)."""
    cfg = ConfigData.model_validate(json.loads((path / "config.json").read_text()), context={"model_id": str(model_id)})
    size = 0
    idx = path / "model.safetensors.index.json"
    if idx.exists():
        size = int((json.loads(idx.read_text()).get("metadata") or {}).get("total_size") or 0)
    if not size:
        size = sum(f.stat().st_size for f in path.glob("*.safetensors"))
    return ModelCard(model_id=model_id, storage_size=Memory.from_bytes(max(size, 1)), n_layers=cfg.layer_count,
                     hidden_size=cfg.hidden_size or 1, supports_tensor=cfg.supports_tensor,
                     num_key_value_heads=cfg.num_key_value_heads, context_length=cfg.max_position_embeddings,
                     tasks=[ModelTask.TextGeneration], trust_remote_code=False, is_custom=True, vision=cfg.vision,
                     backends=list(Backend))


# --------------------------------------------------------------------------------------------
# cache
# --------------------------------------------------------------------------------------------
class CardCache:
    def __init__(self) -> None:
        self.cards: dict[ModelId, ModelCard] = {}
        self.loaded = False

    def _load_dir(self, d: Path, custom: bool) -> None:
        if not d.is_dir():
            return
        for f in sorted(d.rglob("*.toml")):
            try:
                c = ModelCard.load_from_path(f)
            except Exception:  # noqa: BLE001 - a broken card must not take the node down
                continue
            if custom:
                c = c.model_copy(update={"is_custom": True})
            self.cards.setdefault(c.model_id, c)

    def refresh(self) -> None:
        for d in constants.builtin_card_dirs():
            self._load_dir(d, custom=False)
        self._load_dir(constants.EXO_CUSTOM_MODEL_CARDS_DIR, custom=True)
        self.loaded = True

    def get(self, model_id: str) -> ModelCard | None:
        if not self.loaded:
            self.refresh()
        return self.cards.get(ModelId(model_id))

    def list_all(self) -> list[ModelCard]:
        if not self.loaded:
            self.refresh()
        if constants.EXO_ENABLE_IMAGE_MODELS:
            return list(self.cards.values())
        return [c for c in self.cards.values() if not c.is_image]

    def save(self, card: ModelCard) -> None:
        self.cards[card.model_id] = card
        try:
            card.save(constants.EXO_CUSTOM_MODEL_CARDS_DIR / (card.model_id.normalize() + ".toml"))
        except OSError:
            pass

    def pop(self, model_id: str) -> ModelCard | None:
        p = constants.EXO_CUSTOM_MODEL_CARDS_DIR / (ModelId(model_id).normalize() + ".toml")
        try:
            if p.exists():
                p.unlink()
        except OSError:
            pass
        return self.cards.pop(ModelId(model_id), None)


card_cache = CardCache()


def load_card(model_id: str) -> ModelCard:
    """Card for ``model_id``: cache → local checkpoint directory → error (the download layer adds the
    network path: fetch ``config.json`` + index, then call ``card_from_local_dir``)."""
    c = card_cache.get(model_id)
    if c is not None:
        return c
    mid = ModelId(model_id)
    for base in constants.models_dirs():
        p = base / mid.normalize()
        if (p / "config.json").exists():
            c = card_from_local_dir(mid, p)
            card_cache.save(c)
            return c
    if os.path.isdir(model_id) and (Path(model_id) / "config.json").exists():
        c = card_from_local_dir(mid, Path(model_id))
        card_cache.save(c)
        return c
    raise KeyError(f"no model card for {model_id!r} and no local checkpoint to derive one from")
