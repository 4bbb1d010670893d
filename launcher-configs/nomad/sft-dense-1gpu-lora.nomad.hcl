# One GPU, low-rank adapters on a dense model.
job "halo-b200-sft-lora" {
  type = "batch"
  group "trainer" {
    count = 1
    task "train" {
      driver = "docker"
      config {
        image   = "halo-b200:latest"
        command = "python"
        args    = ["-m", "halo_b200.cli", "launch", "sft", "examples/recipes/sft_dense_lora_1gpu.yaml", "-n", "1"]
      }
      resources {
        cpu    = 16000
        memory = 128000
        device "nvidia/gpu" { count = 1 }
      }
    }
  }
}
