from . import llama, puposun, ravapel, rugedra, vofanex  # noqa: F401 (register LlamaForCausalLM, Puposun, Ravapel, Rugedra and Vofanex)
