"""lumen: model interpretability and attribution (the ``tensorplay.lumen`` pack).

Gradient methods (:class:`Saliency`, :class:`InputXGradient`, :class:`IntegratedGradients`,
:class:`GradientShap`, :class:`DeepLift`, :class:`GuidedBackprop`, :class:`Deconvolution`,
:class:`NoiseTunnel`), perturbation and surrogate methods (:class:`FeatureAblation`,
:class:`Occlusion`, :class:`FeaturePermutation`, :class:`ShapleyValues`,
:class:`ShapleyValueSampling`, :class:`Lime`, :class:`KernelShap`), layer methods
(:class:`LayerActivation`, :class:`LayerGradientXActivation`, :class:`LayerGradCam`,
:class:`LayerIntegratedGradients`, :class:`LayerConductance`, :class:`InternalInfluence`,
:class:`NeuronConductance`) and language-model tools (``lumen.llm``: logit lens, activation
patching, attention rollout, gradient attribution of a continuation).

Every algorithm wraps a forward function and exposes ``attribute(inputs, ..., target=...)``; all
of them run on whatever device the model lives on, through autograd and batched forwards.
"""
from . import llm
from ._common import Attribution
from .gradient import (Deconvolution, DeepLift, GradientShap, GuidedBackprop, InputXGradient, IntegratedGradients,
                       NoiseTunnel, Saliency)
from .layer import (InternalInfluence, LayerActivation, LayerAttribution, LayerConductance, LayerGradCam,
                    LayerGradientXActivation, LayerIntegratedGradients, NeuronConductance)
from .llm import LLMGradientAttribution, activation_patching, attention_rollout, logit_lens
from .perturbation import (FeatureAblation, FeaturePermutation, KernelShap, Lime, Occlusion, ShapleyValues,
                           ShapleyValueSampling)
from .variants import (ClassSummarizer, CommonStats, DeepLiftShap, GradientAttribution, GuidedGradCam, LRP,  # noqa: E402
                       LayerDeepLift, LayerFeatureAblation, LayerFeaturePermutation, LayerGradientShap, LayerLRP,
                       NeuronAttribution, NeuronDeconvolution, NeuronDeepLift, NeuronFeatureAblation, NeuronGradient,
                       NeuronGradientShap, NeuronGuidedBackprop, NeuronIntegratedGradients, PerturbationAttribution,
                       Summarizer)
from . import visualization  # noqa: E402
from .extras import (DataLoaderAttribution, GraphDeconvolution, GraphGuidedBackprop, LayerDeepLiftShap, LimeBase,  # noqa: E402
                     NeuronDeepLiftShap, graph_gradient_func, node_names, trace)
from .inputs import (MSE, Count, ImageMaskInput, InterpretableEmbeddingBase, InterpretableInput, LLMAttribution,  # noqa: E402
                     LLMAttributionResult, Max, Mean, Min, ProductBaselines, RemoteLLMAttribution, RemoteLLMProvider, Stat,
                     StatValue, StdDev, Sum, SummarizerSingleTensor, TextTemplateInput, TextTokenInput, TokenReferenceBase, Var,
                     VLLMProvider, configure_interpretable_embedding_layer, remove_interpretable_embedding_layer)

from . import concept, models  # noqa: E402
from .models import (LinearModel, Model, SGDLasso, SGDLinearModel, SGDLinearRegression, SGDRidge, SkLearnLasso,  # noqa: E402
                     SkLearnLinearModel, SkLearnLinearRegression, SkLearnRidge)
_models = models   # the reference's private package name
from .concept import CAV, TCAV, Classifier, Concept, ConceptInterpreter, DefaultClassifier  # noqa: E402
from .llm import (AttributionGraph, AttributionGraphData, CircuitEdge, CircuitNode, FeatureCircuit, FeatureCircuitData,  # noqa: E402
                  GraphEdge, GraphNode, top_attention_heads, top_mlp_features)
from .llm import (CrossLayerTranscoder, collect_component_updates, train_clt, visualize_attention_heads,  # noqa: E402
                  visualize_attention_multi_layer, visualize_token_attention)
from .llm import (ActivationPatching, LogitLens, SparseAutoencoder, collect_hidden_states, extract_attention,  # noqa: E402
                  feature_frequency, reconstruction_error, token_attention, top_activating_indices, train_sae)


def compute_gradients(forward_fn, inputs, target_ind=None, additional_forward_args=None):
    """Gradients of ``forward_fn(*inputs, *additional_forward_args)`` (its ``target_ind`` column when given, summed over
    the batch) with respect to every tensor of ``inputs``: the primitive the gradient methods share
    (lumen/_utils/gradient.py in the reference)."""
    import torch as _torch
    single = isinstance(inputs, _torch.Tensor)
    ins = (inputs,) if single else tuple(inputs)
    extra = () if additional_forward_args is None else (additional_forward_args if isinstance(additional_forward_args, tuple)
                                                         else (additional_forward_args,))
    with _torch.enable_grad():
        ins = tuple(i if i.requires_grad else i.detach().requires_grad_(True) for i in ins)
        out = forward_fn(*ins, *extra)
        if target_ind is not None:
            out = out[:, target_ind] if isinstance(target_ind, int) else out.gather(1, _torch.as_tensor(target_ind).view(-1, 1))[:, 0]
        grads = _torch.autograd.grad(out.sum(), ins)
    return grads[0] if single else grads


InternalAttribution = LayerAttribution   # base of the layer- and neuron-level methods

from .. import _views as _views  # noqa: E402

_views.install(__name__, max_depth=3)
