from . import llama, ravapel, rugedra, vofanex  # noqa: F401 (register LlamaForCausalLM, Ravapel, Rugedra and Vofanex)
