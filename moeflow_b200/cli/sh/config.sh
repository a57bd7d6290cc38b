# Site configuration shared by the shell drivers; every value can be overridden from the environment.
: "${MOEFLOW_PYTHON:=python}"
: "${MOEFLOW_TORCHRUN:=$MOEFLOW_PYTHON -m torch.distributed.run}"
: "${MOEFLOW_VLLM:=vllm}"
: "${MOEFLOW_MODEL_PATH:=checkpoints/GLM-5.3-Flash}"
: "${MOEFLOW_TRIMMED_MODEL_PATH:=checkpoints/GLM-5.3-Flash-4L}"
: "${MOEFLOW_RESULTS_ROOT:=results}"
: "${MOEFLOW_JOBID:=${SLURM_JOB_ID:-local}}"
export MOEFLOW_PYTHON MOEFLOW_TORCHRUN MOEFLOW_VLLM MOEFLOW_MODEL_PATH MOEFLOW_TRIMMED_MODEL_PATH MOEFLOW_RESULTS_ROOT MOEFLOW_JOBID
export MASTER_ADDR=127.0.0.1

# prologue NAME: creates $OUT = results/<name>_<jobid>, logs the command context, refuses busy GPUs
prologue() {
  OUT="$MOEFLOW_RESULTS_ROOT/$1_$MOEFLOW_JOBID"
  mkdir -p "$OUT"
  {
    date -Is
    git rev-parse HEAD 2>/dev/null
    git status --porcelain --untracked-files=no 2>/dev/null | head -20
    nvidia-smi --query-compute-apps=pid,used_memory --format=csv 2>/dev/null
  } >> "$OUT/commands.log"
  export OUT
}
